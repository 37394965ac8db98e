"""out = x . W^T, the matrix product every projection is (src/model.c:299, 302, 307, 309, 324).

float32: CUDA-core kernel with a fixed summation order. bfloat16: the tcgen05
tensor-core kernel where it takes the shape, else the CUDA-core kernel.
"""
import torch

from ..kernels import ops


# Which kernel runs a bfloat16 product of a decode step, measured on a B200 (one launch in a graph, weights from HBM):
# the weight-streaming kernel for a handful of rows has no set-up to speak of (no tensor memory, no barriers) and wins
# where a matrix is one or two round trips to memory: up to 16 rows against matrices of up to 16 MB (all of the
# Qwen3-0.6B shape: 2.9-5.5 us against 5.8-7.9 us), and up to 8 rows against up to 32 MB (the Qwen3-4B shape's q/k/v
# and output projections: 8.2 and 7.8 us against 10.6 and 9.4 us). Beyond that the tensor-memory kernel with its ring
# of TMA stages and K shared out among clusters streams better (4B down projection at 16 rows: 14.7 against 31.8 us;
# 8B shape at 8 rows: 11.5-23.6 us against 14.0-37.6 us), and from 17 rows on it always does.
ROWS_KERNEL_UP_TO = 16
ROWS_KERNEL_BYTES = 16 << 20        # up to ROWS_KERNEL_UP_TO rows
ROWS_KERNEL_BYTES_8 = 32 << 20      # up to 8 rows
GATED_ROWS_KERNEL_BYTES_8 = 128 << 20  # gate/up with the activation in the same kernel: one launch less (4B: 25.4 us
                                       # against 23.0 + 2.5 us at 8 rows; 8B shape, 201 MB: 49.7 against 39.8 + 2.5 us)


def rows_kernel_wins(rows, weight, gated=False):
    nbytes = weight.numel() * weight.element_size()
    if rows > ROWS_KERNEL_UP_TO:
        return False
    return nbytes <= ROWS_KERNEL_BYTES or (rows <= 8 and nbytes <= (GATED_ROWS_KERNEL_BYTES_8 if gated else ROWS_KERNEL_BYTES_8))


class Linear:
    def __init__(self, weight):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def forward(self, x, out, m=None):
        rows = x.shape[0] if m is None else m
        if (self.weight.dtype == torch.bfloat16 and rows_kernel_wins(rows, self.weight)
                and ops.gemm_rows_takes(x, self.weight, out, rows)):
            ops.gemm_rows(x, self.weight, out, rows)
        elif self.weight.dtype == torch.bfloat16 and ops.gemm_tc_takes(x, self.weight, out):
            ops.gemm_tc(x, self.weight, out, m)
        else:
            ops.gemm_simt(x, self.weight, out, m)
        return out
