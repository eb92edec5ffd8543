// Launchers of the statically compiled device kernels (kernels.cu).
#pragma once
#include <cuda_runtime.h>

#include "gemm16.h"

namespace b200 {

struct IGemmLaunch {
  int M, N, K, groups, split_k;
  int Hd, Wd, ldh, ldw;          // dilated input extent and input dilation (masking)
  long long a_sh, a_sw;          // input strides of the two spatial dims
  int a_mcontig, b_kcontig, mask;
  int tensor_cores;              // 1: tcgen05 3xTF32 kernel, 0: fp32 FMA kernel
  int vec;                       // operands can be gathered in uniform, aligned 16-byte chunks
  int seg;                       // vec, and every aligned run of 32 along each operand's contiguous dimension is one 128-byte row
  int tmem_a;                    // with seg: keep the A operand in tensor memory (igemm_tf32x3_ta_kernel)
  int kt_stride;                 // > 0: kt_table holds, per 128-row tile, a count and the k-tiles to visit
  int half_ctas;                 // allow the two-CTAs-per-SM variant of the tensor-memory kernel
  int c_vec;                     // consecutive n are consecutive floats in C (2: and rows start on multiples of four floats)
  int wide_n;                    // use 128-wide N tiles when N >= 128
  // A by TMA (IGemmParams::a_tma): input extents, output row geometry, filter tap geometry
  int a_tma = 0;
  int tma_c = 0, tma_w = 0, tma_h = 0, tma_n = 0, tma_ow = 0, tma_oh = 0, tma_box_h = 0, tma_box_n = 0;
  int tma_kw = 0, tma_pad_h = 0, tma_pad_w = 0, tma_rdil_h = 1, tma_rdil_w = 1;
};

// tables: a_row, a_col, b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp (device pointers).
// `partial` is the split-K scratch ([split_k][groups][M][N] floats) or null when split_k == 1.
// `error_flag` (device int) is counted up by the tensor-core kernel when one of its bounded waits expires.
// Adds the number of kernels launched to *launches.
// `kt_table` (device, may be null): per 128-row tile of M, [count, k-tile indices...] with row length 1 + kt_stride;
// k-tiles outside the list contribute nothing (their rows all fall on padding or dilation holes) and are skipped.
cudaError_t launch_igemm_f32(const IGemmLaunch& p, const void* A, const void* B, void* C, const void* const* tables,
                             void* partial, const int* kt_table, int* error_flag, cudaStream_t stream, int* launches);

}  // namespace b200

namespace b200 {
// Row scatter (stablehlo.scatter with one index along dimension 0 and whole-row updates), deterministic.
// elem_kind: 0 f32, 1 bf16, 2 i32; kind: 0 assign, 1 add, 2 multiply, 3 minimum, 4 maximum. `out` already holds
// the operand; `scratch` has room for scatter_rows_scratch_ints(rows, updates) ints. Updates are ranked by (row, update
// number): all pairs up to 1024 updates, a stable radix sort above.
cudaError_t launch_scatter_rows(int elem_kind, int index_bytes, int kind, long long rows, long long row_elems, int updates,
                                void* out, const void* indices, const void* upd, int* scratch, cudaStream_t stream,
                                int* launches);

// General scatter, second half: `scratch` holds, written by the program's own key kernel, updates destination element
// indices (>= numel: dropped) followed by updates update element indices; they are sorted by destination (stable radix
// sort) and applied run by run in update order. `scratch` has scatter_elems_scratch_ints(updates) ints.
cudaError_t launch_scatter_elems(int elem_kind, int kind, long long numel, int updates, void* out, const void* upd, int* scratch,
                                 cudaStream_t stream, int* launches);

// Split-K fp32 product C[M,N] = A[M,K] * B[K,N] (dense row-major device pointers) whose partial sums go to a
// file-scope device array instead of allocated memory. `*why` explains a refusal. The first call on a device
// resolves the array's device address (cudaGetSymbolAddress); make it before any stream capture.
cudaError_t matmul_f32_static_scratch(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream,
                                      const char** why);
size_t static_scratch_bytes();

// Programmatic stream serialization for the 16-bit product, transpose and repack kernels (on by default).
void set_programmatic_launch(bool on);
void set_igemm_programmatic_launch(bool on);

// One-thread kernels that set the handle of a conditional graph node from device memory: `pred` (one byte) for a while
// node, bounded by `limit_seconds` from the loop's first evaluation (`first` stores the start in *started; when the
// limit passes the loop ends and *error_flag goes up); `index` (i32, out of range = last branch) for a switch node.
cudaError_t launch_while_handle(unsigned long long handle, const void* pred, unsigned long long* started, double limit_seconds,
                                bool first, int* error_flag, cudaStream_t stream);
cudaError_t launch_switch_handle(unsigned long long handle, const void* index, int branches, cudaStream_t stream);

// Test hook: one kernel whose bounded mbarrier wait (budget `polls`) runs out and counts up *error_flag.
cudaError_t launch_expiring_wait(int polls, int* error_flag, cudaStream_t stream);

// TFLOP/s of tcgen05.mma.kind::tf32 (128 x 128 x 8, one CTA per SM, operands resident in shared memory) measured on
// the current device: the fp32-accurate contraction issues three of these per product, so its ceiling is a third.
cudaError_t probe_tf32_mma_rate(int* error_flag, cudaStream_t stream, double* tflops);
}  // namespace b200

namespace b200 {
// Contractions of 16-bit floating-point operands (bf16 or f16) with fp32 accumulation and one rounding to the
// result type: C[g][m][n] = sum_k A(g, m, k) * B(g, k, n), C dense row-major [G][M][N]. Each operand is a strided
// matrix per group with one of its two strides equal to 1 (the reference forwards these to MLX matmul / einsum:
// src/pjrt_plugin/ops/linalg.cc:89-250). Three kernels:
//   path 0  gemm16_tma_kernel : persistent tcgen05.mma kind::f16 tiles of 128 x {64, 128, 256}, operands moved by TMA
//                               tiled copies into 128-byte-swizzled shared memory, accumulators double-buffered in
//                               tensor memory; needs 16-byte aligned bases and strides
//   path 1  gemv16_nc_kernel  : M <= 8 and n contiguous in B: every element of B is read once with 128-bit loads,
//                               K split over warps and CTAs, the last CTA of a column panel adds the splits in order
//   path 2  gemv16_kc_kernel  : M <= 8 and k contiguous in B: one warp per group of output columns, warp-shuffle tree
// Tiled tensor map (128-byte swizzle) over this GPU's memory for TMA copies: `kind` 0 f16, 1 bf16, 2 f32; dims[0] is
// the contiguous dimension, strides_bytes[i] the stride of dims[i + 1]; `map` points at 128 bytes aligned to 64.
bool encode_tensor_map(void* map, int kind, int rank, const void* base, const unsigned long long* dims,
                       const unsigned long long* strides_bytes, const unsigned* box);

// `scratch` (fp32, g.scratch_floats) and `counters` may be null when the plan needs none.
cudaError_t launch_gemm16(const Gemm16Launch& g, const void* A, const void* B, void* C, float* scratch, int* counters,
                          int* error_flag, cudaStream_t stream, int* launches, const char** why);

// dst[b][c][r] = src[b][r][c]: dense source [batch][rows][cols], destination rows `dst_ld` elements apart and batches
// `dst_batch_stride` elements apart (so that several transposes can fill one concatenated tensor), through shared
// memory. Element size 4, or 2 with even extents and 4-byte aligned pointers; anything else returns
// cudaErrorInvalidValue without launching (the caller checks the same conditions when it plans the step).
cudaError_t launch_transpose2d(void* dst, const void* src, int elem_bytes, long long batch, long long rows, long long cols,
                               long long dst_ld, long long dst_batch_stride, cudaStream_t stream, int* launches);

// dst[r][0..cols) = src[r][0..cols) for `rows` rows of 16-bit elements with row strides dst_ld / src_ld (elements): makes
// an operand whose row stride is not a multiple of 16 bytes readable by TMA.
cudaError_t launch_repack_rows16(void* dst, const void* src, long long rows, long long cols, long long dst_ld,
                                 long long src_ld, cudaStream_t stream, int* launches);
}  // namespace b200
