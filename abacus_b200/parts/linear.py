"""out = x . W^T, the matrix product every projection is (src/model.c:299, 302, 307, 309, 324).

float32: CUDA-core kernel with a fixed summation order. bfloat16: the tcgen05
tensor-core kernel where it takes the shape, else the CUDA-core kernel.
"""
import torch

from ..kernels import ops


# Measured on a B200 at the Qwen3-0.6B sizes: up to 16 rows the weight-streaming kernel wins (4-7 us against
# 7.5-8.4 us); at 64 rows every CTA re-reads all of x from the L2 and the tensor-memory kernel wins (13-26 us
# against 21-33 us).
ROWS_KERNEL_UP_TO = 16


class Linear:
    def __init__(self, weight):
        assert weight.dim() == 2 and weight.is_contiguous()
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def forward(self, x, out, m=None):
        rows = x.shape[0] if m is None else m
        # a handful of rows against a matrix too small to give every SM a tensor-memory tile without
        # splitting K: stream the weights through warp-level products instead
        if (self.weight.dtype == torch.bfloat16 and rows <= ROWS_KERNEL_UP_TO and self.out_features <= 32768
                and ops.gemm_rows_takes(x, self.weight, out, rows)):
            ops.gemm_rows(x, self.weight, out, rows)
        elif self.weight.dtype == torch.bfloat16 and ops.gemm_tc_takes(x, self.weight, out):
            ops.gemm_tc(x, self.weight, out, m)
        else:
            ops.gemm_simt(x, self.weight, out, m)
        return out
