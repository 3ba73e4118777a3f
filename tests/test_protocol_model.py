"""The flag protocol of the fused tensor-parallel GEMM kernel, modelled with host threads over shared arrays."""

import pytest

from scaling_b200.parallel.protocol_model import ALLGATHER, ALLREDUCE, REDUCE_SCATTER, ProtocolError, run_sequence

LAYER_FORWARD = [ALLGATHER, REDUCE_SCATTER, ALLGATHER, REDUCE_SCATTER]     # q/k/v, attention out, MLP in, MLP out
LAYER_BACKWARD = [ALLGATHER, REDUCE_SCATTER, REDUCE_SCATTER, ALLGATHER, REDUCE_SCATTER, REDUCE_SCATTER, REDUCE_SCATTER]


@pytest.mark.parametrize("ranks", [2, 4])
@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_a_training_step_worth_of_launches_completes_with_the_right_sums(ranks, seed):
    run_sequence(ranks, LAYER_FORWARD * 2 + LAYER_BACKWARD * 2, seed=seed)


@pytest.mark.parametrize("modes", [[ALLREDUCE] * 6, [ALLREDUCE, ALLGATHER, ALLREDUCE, REDUCE_SCATTER, ALLGATHER, ALLGATHER]])
def test_mixed_modes_share_one_set_of_flags(modes):
    run_sequence(3, modes, seed=5, ctas=4, M=36)


def test_more_ctas_than_tiles_and_a_single_cta():
    run_sequence(2, LAYER_FORWARD, seed=3, ctas=9)
    run_sequence(2, LAYER_FORWARD, seed=4, ctas=1)


def test_a_buffer_is_rewritten_only_two_launches_later_which_is_what_the_alternation_is_for():
    """With a single buffer and no handshake, a rank that is still reading its gathered operand (a linear sharing the
    input) sees it overwritten by a peer that has already started the next all-gather launch."""
    with pytest.raises(ProtocolError, match="gathered operand changed"):
        for seed in range(5):  # the slow reader makes the overlap all but certain; a few seeds make it certain
            run_sequence(2, [ALLGATHER, ALLGATHER], seed=seed, alternate=False, slow_reader=1, M=8, ctas=2)
    for seed in range(3):
        run_sequence(2, [ALLGATHER, ALLGATHER, ALLGATHER], seed=seed, alternate=True, slow_reader=1, M=8, ctas=2)


@pytest.mark.parametrize("ranks", [2, 3])
def test_steps_with_an_odd_number_of_launches_restart_the_alternation(ranks):
    """A replayed step always begins in buffer 0 with a launch that waits for all ranks, whatever buffer the last
    launch of the previous step used."""
    step = [ALLGATHER, REDUCE_SCATTER, ALLGATHER]
    run_sequence(ranks, step * 4, seed=7, step_length=3, slow_reader=ranks - 1)
    run_sequence(ranks, [REDUCE_SCATTER] * 5, seed=8, step_length=1)
