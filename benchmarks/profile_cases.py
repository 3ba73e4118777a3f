"""Small, self-contained workloads of the hot kernels for timing and for profiler captures.

    python -m benchmarks.profile_cases <case> [--iters N]

Each case allocates a few hundred MB at most (inputs larger than the 126 MB L2, so DRAM figures mean something),
runs two warm-up and ``--iters`` timed launches (default 3) with an L2 flush before each timed one, times the launches with CUDA events and
prints one JSON line with the median time and the achieved algorithmic throughput.  The shapes are those of the
125M-parameter decoder at micro batch 8 x 2048 tokens.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch

from scaling_b200.ops import functional as K

TOKENS = 8 * 2048
HIDDEN = 768
HEADS = 12


def _flush_buffer() -> torch.Tensor:
    return torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")


def _time(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(2):  # first calls set kernel attributes, create autograd threads, fill allocator pools
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def case_gemm_fwd(iters: int) -> dict:
    """fc1 forward: [16384, 768] x [3072, 768]^T + bias, GELU, pre-activation kept for the backward pass."""
    x = torch.randn(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(4 * HIDDEN, HIDDEN, device="cuda", dtype=torch.bfloat16) * 0.02
    b = torch.randn(4 * HIDDEN, device="cuda", dtype=torch.bfloat16)
    pre = torch.empty(TOKENS, 4 * HIDDEN, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(pre)
    ms = _time(lambda: K.gemm(x, w, bias=b, act="gelu", pre_act_out=pre, out=out), iters, _flush_buffer())
    flops = 2.0 * TOKENS * HIDDEN * 4 * HIDDEN
    return {"kernel": "gemm_tcgen05 (forward, bias+GELU epilogue)", "ms": ms, "tflops": flops / ms / 1e9,
            "bytes": (x.numel() + w.numel() + 2 * out.numel()) * 2}


def case_gemm_plain(iters: int) -> dict:
    """fc2 forward without epilogue extras: [16384, 3072] x [768, 3072]^T."""
    x = torch.randn(TOKENS, 4 * HIDDEN, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(HIDDEN, 4 * HIDDEN, device="cuda", dtype=torch.bfloat16) * 0.02
    out = torch.empty(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: K.gemm(x, w, out=out), iters, _flush_buffer())
    flops = 2.0 * TOKENS * HIDDEN * 4 * HIDDEN
    return {"kernel": "gemm_tcgen05 (forward)", "ms": ms, "tflops": flops / ms / 1e9,
            "bytes": (x.numel() + w.numel() + out.numel()) * 2}


def case_gemm_fp8(iters: int) -> dict:
    """fc2 forward with e4m3 operands: [16384, 3072] x [768, 3072]^T on the fp8 tensor-core path, bf16 result."""
    x = torch.randn(TOKENS, 4 * HIDDEN, device="cuda").to(torch.float8_e4m3fn)
    w = (torch.randn(HIDDEN, 4 * HIDDEN, device="cuda") * 0.02).to(torch.float8_e4m3fn)
    ms = _time(lambda: K.gemm_fp8(x, w), iters, _flush_buffer())
    flops = 2.0 * TOKENS * HIDDEN * 4 * HIDDEN
    return {"kernel": "gemm_tcgen05 (fp8 operands, kind::f8f6f4)", "ms": ms, "tflops": flops / ms / 1e9,
            "bytes": x.numel() + w.numel() + 2 * TOKENS * HIDDEN}


def case_gemm_fp8_large(iters: int) -> dict:
    """8192 x 8192 x 8192 with e4m3 operands (a compute-bound problem)."""
    n = 8192
    x = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
    w = (torch.randn(n, n, device="cuda") * 0.02).to(torch.float8_e4m3fn)
    ms = _time(lambda: K.gemm_fp8(x, w), iters, _flush_buffer())
    return {"kernel": "gemm_tcgen05 (fp8 operands, kind::f8f6f4)", "ms": ms, "tflops": 2.0 * n ** 3 / ms / 1e9,
            "bytes": 2 * n * n + 2 * n * n}


def case_gemm_wgrad(iters: int) -> dict:
    """fc1 weight gradient: dY^T [3072, 16384] x X [16384, 768], accumulated into the gradient buffer."""
    x = torch.randn(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn(TOKENS, 4 * HIDDEN, device="cuda", dtype=torch.bfloat16)
    dw = torch.zeros(4 * HIDDEN, HIDDEN, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: K.gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True), iters, _flush_buffer())
    flops = 2.0 * TOKENS * HIDDEN * 4 * HIDDEN
    return {"kernel": "gemm_tcgen05 (weight gradient, split-K)", "ms": ms, "tflops": flops / ms / 1e9,
            "bytes": (x.numel() + dy.numel() + 2 * dw.numel()) * 2}


def _attention_inputs():
    qkv = torch.randn(TOKENS, HEADS, 3 * 64, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, TOKENS + 1, 2048, device="cuda", dtype=torch.int32)
    pos = torch.arange(2048, device="cuda", dtype=torch.int32).repeat(8)
    return qkv, cu, pos


def case_attention_fwd(iters: int) -> dict:
    """Causal self-attention forward on the packed projection, 8 documents of 2048 tokens, 12 heads of 64."""
    from scaling_b200.ops.attention_kernel import packed_qkv_attention

    qkv, cu, pos = _attention_inputs()
    with torch.no_grad():
        ms = _time(lambda: packed_qkv_attention(qkv.clone(), pos, (64, 10000.0, False), cu, True, 0.125, None), iters,
                   _flush_buffer())
    flops = 4.0 * 8 * HEADS * 2048 * 2048 * 64 / 2
    return {"kernel": "fa_fwd_kernel<64> (+ rope, clone)", "ms": ms, "tflops": flops / ms / 1e9, "bytes": qkv.numel() * 2}


def case_attention_bwd(iters: int) -> dict:
    """Forward + backward of the same attention (backward = delta, dK/dV, dQ kernels and the inverse rotation)."""
    from scaling_b200.ops.attention_kernel import packed_qkv_attention

    qkv, cu, pos = _attention_inputs()
    src = qkv.requires_grad_()
    do = torch.randn(TOKENS, HEADS, 64, device="cuda", dtype=torch.bfloat16)

    def run():
        out = packed_qkv_attention(src * 1.0, pos, (64, 10000.0, False), cu, True, 0.125, None)
        out.backward(do)

    ms = _time(run, iters, _flush_buffer())
    flops = 3.5 * 4.0 * 8 * HEADS * 2048 * 2048 * 64 / 2
    return {"kernel": "fa_fwd + fa_bwd_dkdv + fa_bwd_dq <64>", "ms": ms, "tflops": flops / ms / 1e9,
            "bytes": qkv.numel() * 2 * 3}


def case_attention_fwd_d64(iters: int) -> dict:
    """The forward kernel alone at head size 64 (separate q, k, v; no rotary embedding, no copies)."""
    from scaling_b200.ops.attention import flash_attention

    q, k, v = (torch.randn(TOKENS, HEADS, 64, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    cu = torch.arange(0, TOKENS + 1, 2048, device="cuda", dtype=torch.int32)
    with torch.no_grad():
        ms = _time(lambda: flash_attention(q, k, v, cu, None, causal=True), iters, _flush_buffer())
    flops = 4.0 * 8 * HEADS * 2048 * 2048 * 64 / 2
    return {"kernel": "fa_fwd_kernel<64>", "ms": ms, "tflops": flops / ms / 1e9, "bytes": 4 * q.numel() * 2}


def _attention_inputs_d128():
    """Two documents of 4096 tokens, 16 query / 4 key-value heads of 128 (the 7B model on two tensor-parallel ranks)."""
    T, hq, hkv = 2 * 4096, 16, 4
    q = torch.randn(T, hq, 128, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(T, hkv, 128, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(T, hkv, 128, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(0, T + 1, 4096, device="cuda", dtype=torch.int32)
    return q, k, v, cu, 4.0 * 2 * hq * 4096 * 4096 * 128 / 2


def case_attention_fwd_d128(iters: int) -> dict:
    """Causal grouped-query attention forward at head size 128."""
    from scaling_b200.ops.attention import flash_attention

    q, k, v, cu, flops = _attention_inputs_d128()
    with torch.no_grad():
        ms = _time(lambda: flash_attention(q, k, v, cu, None, causal=True), iters, _flush_buffer())
    return {"kernel": "fa_fwd_kernel<128>", "ms": ms, "tflops": flops / ms / 1e9,
            "bytes": (2 * q.numel() + 2 * k.numel()) * 2}


def case_attention_bwd_d128(iters: int) -> dict:
    """Forward + backward of the same attention (backward = delta, dK/dV with the head group split, dQ)."""
    from scaling_b200.ops.attention import flash_attention

    q, k, v, cu, flops = _attention_inputs_d128()
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    do = torch.randn_like(q)

    def run():
        flash_attention(q, k, v, cu, None, causal=True).backward(do)
        q.grad = k.grad = v.grad = None

    ms = _time(run, iters, _flush_buffer())
    return {"kernel": "fa_fwd + fa_bwd_dkdv + fa_bwd_dq <128>", "ms": ms, "tflops": 3.5 * flops / ms / 1e9,
            "bytes": (4 * q.numel() + 4 * k.numel()) * 2}


def case_norm(iters: int) -> dict:
    """LayerNorm forward + backward on [16384, 768]."""
    x = torch.randn(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.ones(HIDDEN, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    b = torch.zeros(HIDDEN, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(TOKENS, HIDDEN, device="cuda", dtype=torch.bfloat16)

    def run():
        K.layer_norm(x, w, b, 1e-5).backward(dy)

    ms = _time(run, iters, _flush_buffer())
    nbytes = TOKENS * HIDDEN * 2 * 5  # x, y, dy, x again, dx
    return {"kernel": "norm_fwd_kernel + norm_bwd_warp_kernel", "ms": ms, "gbs": nbytes / ms / 1e6, "bytes": nbytes}


def case_adamw(iters: int) -> dict:
    """Fused AdamW on 64M fp32 master weights with bf16 gradients and the bf16 write-out."""
    n = 64 * 1024 * 1024
    p = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    lp = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ms = _time(lambda: K.adamw_step(p, m, v, g, lp, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1), iters, _flush_buffer())
    nbytes = n * (3 * 8 + 2 + 2)
    return {"kernel": "adamw_kernel", "ms": ms, "gbs": nbytes / ms / 1e6, "bytes": nbytes}


CASES = {"gemm_fp8": case_gemm_fp8, "gemm_fp8_large": case_gemm_fp8_large, "gemm_fwd": case_gemm_fwd, "gemm_plain": case_gemm_plain, "gemm_wgrad": case_gemm_wgrad,
         "attention_fwd": case_attention_fwd, "attention_bwd": case_attention_bwd,
         "attention_fwd_d64": case_attention_fwd_d64, "attention_fwd_d128": case_attention_fwd_d128, "attention_bwd_d128": case_attention_bwd_d128, "norm": case_norm,
         "adamw": case_adamw}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        sys.exit("a CUDA device is required")
    out = CASES[args.case](args.iters)
    K.check_status()
    out["case"] = args.case
    print(json.dumps(out))


if __name__ == "__main__":
    main()
