"""GEMM + epilogue fusion pass (placeholder until the tcgen05 GEMM lands)."""


def fuse_gemm_epilogues(gm) -> int:
    return 0
