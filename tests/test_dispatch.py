"""Which kernel a decode product goes to, by rows and matrix size (no GPU: the choice is host code)."""
import pytest
import torch

from herbert_rs_b200 import ops


def kernel_for(M, N, K):
    a = torch.empty(M, K, dtype=torch.bfloat16)
    w = torch.empty(1, K, dtype=torch.bfloat16).expand(N, K)       # only the shape matters here: no memory behind the rows
    return ops._decode_gemm(a, w).__name__


SHAPES_8B = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (24576, 4096), "down": (4096, 12288), "head": (151936, 4096)}
SHAPES_06B = {"qkv": (4096, 1024), "o": (1024, 2048), "gate_up": (6144, 1024), "down": (1024, 3072)}
SHAPES_32B = {"qkv": (10240, 5120), "o": (5120, 8192), "gate_up": (51200, 5120), "down": (5120, 25600)}


@pytest.mark.parametrize("M", [1, 8, 16])
def test_up_to_sixteen_rows_everything_streams_through_the_mma_sync_kernel(M):
    for shapes in (SHAPES_8B, SHAPES_06B, SHAPES_32B):
        for N, K in shapes.values():
            assert kernel_for(M, N, K) == "gemm_skinny"


def test_mid_batches_at_8b_sizes():
    for M in (17, 32):
        assert kernel_for(M, *SHAPES_8B["qkv"]) == "gemm_tcgen05"
        assert kernel_for(M, *SHAPES_8B["gate_up"]) == "gemm_tcgen05"
        assert kernel_for(M, *SHAPES_8B["o"]) == "gemm_skinny"
        assert kernel_for(M, *SHAPES_8B["down"]) == "gemm_skinny"
        assert kernel_for(M, *SHAPES_8B["head"]) == "gemm_stream"
    for M in (33, 64):
        assert kernel_for(M, *SHAPES_8B["down"]) == "gemm_tcgen05"
        assert kernel_for(M, *SHAPES_8B["o"]) == "gemm_skinny"
        assert kernel_for(M, *SHAPES_8B["head"]) == "gemm_stream"


def test_mid_batches_at_other_sizes():
    for M in (17, 64):
        for N, K in SHAPES_06B.values():
            assert kernel_for(M, N, K) == "gemm_skinny"          # matrices of a few MB: the fixed cost decides
    for name, (N, K) in SHAPES_32B.items():
        assert kernel_for(64, N, K) == "gemm_tcgen05"
    assert kernel_for(32, *SHAPES_32B["down"]) == "gemm_tcgen05"  # 131 M elements
    assert kernel_for(32, *SHAPES_32B["o"]) == "gemm_skinny"      # 42 M elements, 5,120 rows
