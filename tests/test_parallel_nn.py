"""Tensor-parallel building blocks on CPU ranks (gloo) against their plain PyTorch counterparts."""

import pytest
import torch

from tests.test_core_distributed import _topology
from tests.utils import dist_launcher

pytestmark = pytest.mark.dist


def _full_weight(shards, dim):
    return torch.cat(shards, dim=dim)


# ---------------------------------------------------------------------------------------------- linears
def _linear_worker(rank, world_size, port, device, in_features, out_features, sp):
    from scaling_b200.core.nn.linear import ColumnParallelLinear, RowParallelLinear
    from scaling_b200.core.utils.param_merge import merge_parameter

    t = _topology(rank, world_size, port, mp=world_size)
    torch.manual_seed(5)
    x = torch.randn(2, 6, in_features)
    out = {}
    for cls, kw in ((ColumnParallelLinear, dict(parallel_output=False)), (RowParallelLinear, dict(parallel_input=False))):
        layer = cls(in_features=in_features, out_features=out_features, bias=True, topology=t,
                    init_method=lambda w: torch.nn.init.normal_(w, std=0.1), **kw)
        torch.nn.init.normal_(layer.bias, std=0.1)
        if cls is RowParallelLinear and world_size > 1:  # the bias is replicated: same values on every rank
            torch.distributed.broadcast(layer.bias.data, 0)
        xin = x.clone().requires_grad_()
        y = layer(xin)
        y.square().sum().backward()
        weight = merge_parameter(layer.weight, layer.weight.core_parameter_meta, t)
        bias = merge_parameter(layer.bias, layer.bias.core_parameter_meta, t)
        ref_in = x.clone().requires_grad_()
        ref = torch.nn.functional.linear(ref_in, weight, bias)
        ref.square().sum().backward()
        out[cls.__name__] = ((y - ref).abs().max().item(), (xin.grad - ref_in.grad).abs().max().item())
    return out


@pytest.mark.parametrize("world_size", [1, 2])
@pytest.mark.parametrize("in_features,out_features", [(8, 8), (16, 32), (32, 16)])
def test_parallel_linears_equal_a_plain_linear(world_size, in_features, out_features):
    for per_rank in dist_launcher(_linear_worker, world_size, in_features=in_features, out_features=out_features, sp=False):
        for name, (dy, dx) in per_rank.items():
            assert dy < 1e-5 and dx < 1e-4, (name, dy, dx)


# ---------------------------------------------------------------------------------------------- embedding
def _embedding_worker(rank, world_size, port, device):
    from scaling_b200.core.nn.linear import VocabParallelEmbedding
    from scaling_b200.core.utils.param_merge import merge_parameter

    t = _topology(rank, world_size, port, mp=world_size)
    torch.manual_seed(7)
    emb = VocabParallelEmbedding(num_embeddings=32, embedding_dim=8, topology=t, finetunable_token_ids=[3, 20],
                                 init_method=lambda w: torch.nn.init.normal_(w, std=1.0))
    ids = torch.tensor([[0, 3, 15, 16], [20, 31, 3, 3]])
    y = emb(ids)
    y.sum().backward()
    full = merge_parameter(emb.weight, emb.weight.core_parameter_meta, t)
    ref = torch.nn.functional.embedding(ids, full)
    grad_rows = emb.weight.grad.abs().sum(dim=1).nonzero().flatten() + emb.vocab_start_index
    return (y - ref).abs().max().item(), sorted(grad_rows.tolist())


@pytest.mark.parametrize("world_size", [1, 2])
def test_vocab_parallel_embedding_and_finetunable_rows(world_size):
    results = dist_launcher(_embedding_worker, world_size)
    trained = sorted({r for _, rows in results for r in rows})
    assert all(err < 1e-6 for err, _ in results)
    assert trained == [3, 20]  # gradients reach the listed token ids only


# ---------------------------------------------------------------------------------------------- rotary (no ranks)
def test_rotary_forms_agree_after_layout_translation():
    from scaling_b200.core.nn.rotary import RotaryConfig, RotaryEmbedding, RotaryEmbeddingComplex

    torch.manual_seed(0)
    s, b, h, d = 6, 2, 3, 8
    q, k = torch.randn(s, b, h, d), torch.randn(s, b, h, d)
    half, cplx = RotaryEmbedding(RotaryConfig(dimensions=d)), RotaryEmbeddingComplex(RotaryConfig(dimensions=d))
    # rotate-half pairs (i, i + d/2); the complex form pairs (2i, 2i + 1): permute the head dimension between them
    perm = torch.arange(d).view(2, d // 2).t().reshape(-1)  # position 2i <- i, 2i+1 <- i + d/2
    qh, kh = half(q, k)
    qc, kc = cplx(q[..., perm], k[..., perm])
    assert torch.allclose(qh[..., perm], qc, atol=1e-5) and torch.allclose(kh[..., perm], kc, atol=1e-5)
    # the attention scores do not depend on the form
    assert torch.allclose(torch.einsum("sbhd,tbhd->bhst", qh, kh), torch.einsum("sbhd,tbhd->bhst", qc, kc), atol=1e-4)


def test_rotary_position_ids_shift_the_rotation_and_partial_dims_pass_through():
    from scaling_b200.core.nn.rotary import RotaryConfig, RotaryEmbedding

    torch.manual_seed(0)
    s, b, h, d = 5, 1, 2, 8
    x = torch.randn(s, b, h, d)
    rot = RotaryEmbedding(RotaryConfig(dimensions=4))
    plain, _ = rot(x, x)
    shifted, _ = rot(x, x, query_position_ids=torch.arange(3, 3 + s).view(s, 1))
    again, _ = rot(x[:2], x[:2], query_position_ids=torch.tensor([[3], [4]]))
    assert torch.equal(plain[..., 4:], x[..., 4:])  # only the first `dimensions` entries rotate
    assert torch.allclose(plain[0], x[0], atol=1e-6)  # position 0 is the identity
    assert torch.allclose(shifted[:2], again, atol=1e-6) and not torch.allclose(shifted, plain)
    # relative property: scores depend on position differences only
    q0, k0 = rot(x, x)
    q3, k3 = rot(x, x, torch.arange(3, 3 + s).view(s, 1), torch.arange(3, 3 + s).view(s, 1))
    assert torch.allclose(torch.einsum("sbhd,tbhd->bhst", q0, k0), torch.einsum("sbhd,tbhd->bhst", q3, k3), atol=1e-4)


# ---------------------------------------------------------------------------------------------- norms / softmax
@pytest.mark.parametrize("rms", [False, True])
def test_norms_match_their_definitions(rms):
    from scaling_b200.core.nn.norm import LayerNormConfig, NormType, get_norm

    torch.manual_seed(1)
    x = torch.randn(3, 5, 16, requires_grad=True)
    norm = get_norm(norm_type=NormType.RMS if rms else NormType.LAYERNORM, layernorm_config=LayerNormConfig(),
                    dimensions=16, device=torch.device("cpu"), dtype=torch.float32)
    torch.nn.init.normal_(norm.weight, mean=1.0, std=0.1)
    y = norm(x)
    eps = norm.config.layernorm_epsilon if hasattr(norm, "config") else 1e-5
    if rms:
        ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + getattr(norm, "eps", eps)) * norm.weight
    else:
        ref = torch.nn.functional.layer_norm(x, (16,), norm.weight, norm.bias, eps)
    assert torch.allclose(y, ref, atol=1e-5)
    y.sum().backward()
    assert x.grad is not None and norm.weight.grad is not None


def test_masked_softmax_kernels_agree():
    from scaling_b200.core.nn.masked_softmax import MaskedSoftmax, MaskedSoftmaxConfig, MaskedSoftmaxKernel

    torch.manual_seed(2)
    scores = torch.randn(2, 3, 6, 6)
    mask = torch.triu(torch.ones(6, 6, dtype=torch.bool), 1).view(1, 1, 6, 6).expand(2, 1, 6, 6)
    outs = []
    for kernel in MaskedSoftmaxKernel:
        for fp32 in (True, False):
            m = MaskedSoftmax(MaskedSoftmaxConfig(kernel=kernel, softmax_in_fp32=fp32, scale=0.5))
            outs.append(m(scores.clone(), mask))
    ref = torch.softmax((scores * 0.5).masked_fill(mask, -10000.0), dim=-1)
    for o in outs:
        assert torch.allclose(o, ref, atol=1e-6)


# ---------------------------------------------------------------------------------------------- LoRA
def _lora_worker(rank, world_size, port, device, qkv_in_one, kv_heads):
    from scaling_b200.core.nn.attention import ParallelSelfAttention
    from scaling_b200.core.nn.lora import LoRaConfig
    from scaling_b200.core.nn.masked_softmax import MaskedSoftmaxConfig
    from scaling_b200.core.nn.rotary import RotaryConfig

    t = _topology(rank, world_size, port, mp=world_size)
    torch.manual_seed(3)
    lora = LoRaConfig(name="l", rank=2, alpha=4, parallel_modules=["query", "key", "value", "dense"])
    attn = ParallelSelfAttention(hidden_size=32, num_attention_heads=4, masked_softmax_config=MaskedSoftmaxConfig(),
                                 topology=t, lora_config=lora, qkv_in_one=qkv_in_one, num_kv_heads=kv_heads,
                                 rotary_config=RotaryConfig(dimensions=8),
                                 init_method=lambda w: torch.nn.init.normal_(w, std=0.2))
    for p in attn.lora_modules.parameters():  # the B matrices start at zero: give the adapters an effect
        torch.nn.init.normal_(p, std=0.3)
    torch.manual_seed(11)
    x = torch.randn(2, 8, 32)
    cu = torch.tensor([0, 8, 16], dtype=torch.int32)
    weights_before = {n: p.detach().clone() for n, p in attn.named_parameters() if "lora" not in n and n.endswith("weight")}
    with torch.no_grad():
        y_adapters = attn(x, cumulative_seq_lengths=cu, position_ids=None)
        attn.merge_lora_weights()
        y_merged = attn(x, cumulative_seq_lengths=cu, position_ids=None)
    changed = [n for n, p in attn.named_parameters() if n in weights_before and not torch.equal(p, weights_before[n])]
    still_lora = any("lora" in n for n, _ in attn.named_parameters())
    return (y_adapters - y_merged).abs().max().item(), y_adapters.abs().mean().item(), len(changed), still_lora


@pytest.mark.parametrize("world_size", [1, 2])
@pytest.mark.parametrize("qkv_in_one,kv_heads", [(True, None), (False, 2)])
def test_lora_merge_keeps_the_output_and_changes_the_weights(world_size, qkv_in_one, kv_heads):
    for err, scale, changed, has_lora in dist_launcher(_lora_worker, world_size, qkv_in_one=qkv_in_one, kv_heads=kv_heads):
        assert err < 1e-4 * max(1.0, scale), (err, scale)
        assert changed >= 2 and not has_lora


# ---------------------------------------------------------------------------------------------- fp8 linear (no ranks)
def test_fp8_linear_stays_close_to_the_full_precision_linear():
    from scaling_b200.core.fp8.fp8_linear import fp8_linear

    torch.manual_seed(0)
    x = torch.randn(16, 64, requires_grad=True)
    w = (torch.randn(32, 64) * 0.2).requires_grad_()
    b = torch.randn(32, requires_grad=True)
    e4, e5 = torch.float8_e4m3fn, torch.float8_e5m2
    y = fp8_linear(x, w, b, dtypes_forward=(e4, e4), dtypes_grad_input=(e5, e4), dtypes_grad_weight=(e4, e5))
    y.square().mean().backward()
    got = (y.detach(), x.grad.clone(), w.grad.clone(), b.grad.clone())
    x.grad = w.grad = b.grad = None
    ref = torch.nn.functional.linear(x, w, b)
    ref.square().mean().backward()
    for g, r in zip(got, (ref.detach(), x.grad, w.grad, b.grad)):
        assert (g - r).norm() / r.norm() < 0.1
    assert not torch.equal(got[0], ref.detach())  # the operands were rounded
    # saturation instead of inf: values beyond the format's range clamp to its maximum
    big = fp8_linear(torch.full((1, 4), 1e6), torch.eye(4), None, dtypes_forward=(e4, e4))
    assert torch.isfinite(big).all() and big.max() == torch.finfo(e4).max
    # a product without a dtype pair runs unquantised; left out, the pairs default to the ones used above
    assert torch.allclose(fp8_linear(x, w, b, None, None, None), ref)
    assert torch.equal(fp8_linear(x, w, b), y)


def test_key_ranges_of_cross_length_attention_match_the_dense_mask():
    """The per-query key ranges that the decode kernel reads describe exactly the mask of the dense expression, for
    queries shorter and longer than the keys, causal or not, with and without a local window."""
    import itertools

    from scaling_b200.ops.attention import attention_mask_from_cu_seqlens
    from scaling_b200.ops.attention_kernel import key_ranges

    gen = torch.Generator().manual_seed(5)
    for trial in range(60):
        docs = int(torch.randint(1, 4, (1,), generator=gen))
        len_q = torch.randint(1, 6, (docs,), generator=gen)
        len_k = len_q + torch.randint(0, 9, (docs,), generator=gen)
        if trial % 5 == 0:
            len_k = torch.maximum(len_q - 2, torch.ones_like(len_q))  # fewer keys than queries
        cu_q = torch.cat([torch.zeros(1, dtype=torch.long), len_q.cumsum(0)]).int()
        cu_k = torch.cat([torch.zeros(1, dtype=torch.long), len_k.cumsum(0)]).int()
        tq, tk = int(cu_q[-1]), int(cu_k[-1])
        for causal, window in itertools.product((True, False), (None, 0, 2, 100)):
            allowed = attention_mask_from_cu_seqlens(cu_q, cu_k, tq, tk, causal, window)
            lo, hi = key_ranges(cu_q, cu_k, tq, causal, window)
            keys = torch.arange(tk)[None]
            assert torch.equal(allowed, (keys >= lo[:, None]) & (keys < hi[:, None])), (cu_q, cu_k, causal, window)
