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


def test_pushing_before_the_peer_has_entered_is_what_the_entry_flags_prevent():
    """Without the rule, a rank that is still reading its gathered operand (a linear sharing the input) sees it
    overwritten by a peer that has already started the next all-gather launch."""
    with pytest.raises(ProtocolError, match="gathered operand changed"):
        for seed in range(5):  # the slow reader makes the overlap all but certain; a few seeds make it certain
            run_sequence(2, [ALLGATHER, ALLGATHER], seed=seed, wait_for_entry=False, slow_reader=1, M=8, ctas=2)
    run_sequence(2, [ALLGATHER, ALLGATHER], seed=0, wait_for_entry=True, slow_reader=1, M=8, ctas=2)
