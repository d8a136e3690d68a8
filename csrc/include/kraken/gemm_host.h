// Host-side helpers shared by the GEMM translation units: the tensor-map cache, tiling defaults
// and the operand set-up of C[M,N] = A[M,K] * Bt[N,K]^T. Defined in gemm.cu.
#pragma once
#include "kraken/driver_api.h"
#include "kraken/gemm_core.cuh"

namespace kraken {

// Tensor map of a row-major bf16 (elt 2) or fp32 (elt 4) matrix [rows, cols] (cols contiguous, `ld`
// elements per row), box = 128 bytes of columns x box_rows rows, 128-byte swizzle, out-of-range
// elements read as zero. Cached.
int get_tmap(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
             unsigned box_rows, CUtensorMap* out, int elt = 2);
// Tensor map for TMA stores of bf16 tiles (box of 32 rows); false when the matrix cannot be
// described to TMA or TMA stores are switched off.
bool store_tmap(const void* ptr, long long rows, long long cols, long long ld, CUtensorMap* m);
int default_group_r();
bool pair_enabled();
unsigned grid_cap(const DeviceState* d);
int setup_problem(GemmParams& p, const void* a, long long lda, const void* bt, long long ldb, int M, int N, int K,
                  bool swap, int bn_override, int* bn_out, int elt = 2);
// Single-CTA kernels for fp32 operands multiplied as tf32 (plain GEMM and GEMM -> all-reduce;
// column tiles of 16, 64 or 256). Defined in gemm_tf32.cu.
int launch_gemm_tf32(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream);
// Single-CTA kernels of the decode GEMM -> all-reduce. Defined in gemm_ar.cu.
int launch_gemm_ar(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream);
// Routes a parameter block to the kernel family of its mode and operand type (gemm.cu).
int launch_gemm(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream);
int pick_bn(int rows_c);      // column-tile width for `rows_c` rows of the column operand
int tf32_bn(int rows_c);      // the same among the widths the tf32 kernels exist for

}  // namespace kraken
