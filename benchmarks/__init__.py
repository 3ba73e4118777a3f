"""Micro-benchmarks and profiler workloads of the kernels (not part of the importable library).

``python -m benchmarks.profile_cases <case>`` runs one kernel on one shape (the commands in ``profiles/*.md``);
``torchrun --nproc-per-node N -m benchmarks.fused_tp`` times the fused tensor-parallel GEMMs against GEMM + NCCL.
"""
