// Hand-written device kernels that are not generated per program: the
// table-driven implicit GEMM behind stablehlo.convolution and
// stablehlo.dot_general (the reference forwards these to MLX:
// src/pjrt_plugin/ops/linalg.cc:89-250 dot_general, :253-550 convolution) and
// its split-K reduction.
//
// C[g][m][n] = sum_k A(g, m, k) * B(g, k, n), fp32 operands, fp32 FMA
// accumulation (no TF32 rounding anywhere). Every index goes through a table
// built at compile time, so one kernel serves forward convolution, the
// input-gradient form (lhs_dilation, negative padding), the kernel-gradient
// form (batch as contraction, rhs_dilation) and any dot_general layout:
//   A address = a_grp[g] + a_row[m].off + a_col[k].off + (ih / ldh) * a_sh + (iw / ldw) * a_sw
//     with ih = a_row[m].h0 + a_col[k].dh, iw = a_row[m].w0 + a_col[k].dw; the element is zero unless
//     0 <= ih < Hd, 0 <= iw < Wd, ih % ldh == 0 and iw % ldw == 0   (dilate, then pad: linalg.cc:508-532)
//   B address = b_grp[g] + b_row[k] + b_col[n]
//   C address = c_grp[g] + c_row[m] + c_col[n]
#include <cuda_runtime.h>

#include "kernels.h"

namespace b200 {

namespace {

constexpr int BM = 128, BN = 64, BK = 16, NT = 256;
constexpr int TM = 8, TN = 4;

struct RowEnt { long long off; int h0, w0; };
struct ColEnt { long long off; int dh, dw; };

template <bool A_MCONTIG, bool B_KCONTIG, bool MASK>
__global__ void __launch_bounds__(NT) igemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                       float* __restrict__ C, const RowEnt* __restrict__ a_row,
                                                       const ColEnt* __restrict__ a_col,
                                                       const long long* __restrict__ b_row,
                                                       const long long* __restrict__ b_col,
                                                       const long long* __restrict__ c_row,
                                                       const long long* __restrict__ c_col,
                                                       const long long* __restrict__ a_grp,
                                                       const long long* __restrict__ b_grp,
                                                       const long long* __restrict__ c_grp, float* __restrict__ partial,
                                                       IGemmLaunch p) {
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int g = blockIdx.z / p.split_k, sp = blockIdx.z % p.split_k;
  const int kchunk = ((p.K + p.split_k - 1) / p.split_k + BK - 1) / BK * BK;
  const int kbeg = sp * kchunk, kend = min(p.K, kbeg + kchunk);
  const float* Ag = A + a_grp[g];
  const float* Bg = B + b_grp[g];

  // which elements of the A and B tiles this thread fetches
  constexpr int A_PER = BM * BK / NT, B_PER = BK * BN / NT;
  RowEnt rows[A_MCONTIG ? 1 : A_PER];
  bool row_ok[A_MCONTIG ? 1 : A_PER];
  if (A_MCONTIG) {
    int m = m0 + tid % BM;
    row_ok[0] = m < p.M;
    rows[0] = row_ok[0] ? a_row[m] : RowEnt{0, 0, 0};
  } else {
#pragma unroll
    for (int i = 0; i < A_PER; i++) {
      int m = m0 + tid / BK + (NT / BK) * i;
      row_ok[i] = m < p.M;
      rows[i] = row_ok[i] ? a_row[m] : RowEnt{0, 0, 0};
    }
  }
  long long bcols[B_KCONTIG ? B_PER : 1];
  bool bcol_ok[B_KCONTIG ? B_PER : 1];
  if (B_KCONTIG) {
#pragma unroll
    for (int i = 0; i < B_PER; i++) {
      int n = n0 + tid / BK + (NT / BK) * i;
      bcol_ok[i] = n < p.N;
      bcols[i] = bcol_ok[i] ? b_col[n] : 0;
    }
  } else {
    int n = n0 + tid % BN;
    bcol_ok[0] = n < p.N;
    bcols[0] = bcol_ok[0] ? b_col[n] : 0;
  }

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = 0.f;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);

  auto fetch_a = [&](const RowEnt& r, bool rok, const ColEnt& c, bool cok) -> float {
    if (!rok || !cok) return 0.f;
    if (MASK) {
      int ih = r.h0 + c.dh, iw = r.w0 + c.dw;
      if (ih < 0 || iw < 0 || ih >= p.Hd || iw >= p.Wd) return 0.f;
      if (p.ldh != 1) { if (ih % p.ldh) return 0.f; ih /= p.ldh; }
      if (p.ldw != 1) { if (iw % p.ldw) return 0.f; iw /= p.ldw; }
      return __ldg(Ag + r.off + c.off + (long long)ih * p.a_sh + (long long)iw * p.a_sw);
    }
    return __ldg(Ag + r.off + c.off);
  };

  for (int k0 = kbeg; k0 < kend; k0 += BK) {
    float ra[A_PER], rb[B_PER];
    if (A_MCONTIG) {
#pragma unroll
      for (int i = 0; i < A_PER; i++) {
        int k = k0 + tid / BM + (NT / BM) * i;
        bool cok = k < kend;
        ColEnt c = cok ? a_col[k] : ColEnt{0, 0, 0};
        ra[i] = fetch_a(rows[0], row_ok[0], c, cok);
      }
    } else {
      int k = k0 + tid % BK;
      bool cok = k < kend;
      ColEnt c = cok ? a_col[k] : ColEnt{0, 0, 0};
#pragma unroll
      for (int i = 0; i < A_PER; i++) ra[i] = fetch_a(rows[i], row_ok[i], c, cok);
    }
    if (B_KCONTIG) {
      int k = k0 + tid % BK;
      bool kok = k < kend;
      long long br = kok ? b_row[k] : 0;
#pragma unroll
      for (int i = 0; i < B_PER; i++) rb[i] = (kok && bcol_ok[i]) ? __ldg(Bg + br + bcols[i]) : 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < B_PER; i++) {
        int k = k0 + tid / BN + (NT / BN) * i;
        bool kok = k < kend;
        rb[i] = (kok && bcol_ok[0]) ? __ldg(Bg + b_row[kok ? k : 0] + bcols[0]) : 0.f;
      }
    }
    __syncthreads();
    if (A_MCONTIG) {
#pragma unroll
      for (int i = 0; i < A_PER; i++) As[tid / BM + (NT / BM) * i][tid % BM] = ra[i];
    } else {
#pragma unroll
      for (int i = 0; i < A_PER; i++) As[tid % BK][tid / BK + (NT / BK) * i] = ra[i];
    }
    if (B_KCONTIG) {
#pragma unroll
      for (int i = 0; i < B_PER; i++) Bs[tid % BK][tid / BK + (NT / BK) * i] = rb[i];
    } else {
#pragma unroll
      for (int i = 0; i < B_PER; i++) Bs[tid / BN + (NT / BN) * i][tid % BN] = rb[i];
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float a[TM], b[TN];
      const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * TM]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][ty * TM + 4]);
      a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
      a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[kk][tx * TN]);
      b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
  }

  if (p.split_k > 1) {
    float* out = partial + ((long long)sp * p.groups + g) * (long long)p.M * p.N;
#pragma unroll
    for (int i = 0; i < TM; i++) {
      int m = m0 + ty * TM + i;
      if (m >= p.M) continue;
#pragma unroll
      for (int j = 0; j < TN; j++) {
        int n = n0 + tx * TN + j;
        if (n < p.N) out[(long long)m * p.N + n] = acc[i][j];
      }
    }
  } else {
    float* Cg = C + c_grp[g];
    long long cc[TN];
#pragma unroll
    for (int j = 0; j < TN; j++) {
      int n = n0 + tx * TN + j;
      cc[j] = n < p.N ? c_col[n] : -1;
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
      int m = m0 + ty * TM + i;
      if (m >= p.M) continue;
      long long cr = c_row[m];
#pragma unroll
      for (int j = 0; j < TN; j++)
        if (cc[j] >= 0) Cg[cr + cc[j]] = acc[i][j];
    }
  }
}

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ C,
                                                            const long long* __restrict__ c_row,
                                                            const long long* __restrict__ c_col,
                                                            const long long* __restrict__ c_grp, int M, int N, int groups,
                                                            int split_k) {
  long long total = (long long)groups * M * N;
  long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int k = 0; k < split_k; k++) s += partial[(long long)k * total + i];
  int n = (int)(i % N);
  int m = (int)((i / N) % M);
  int g = (int)(i / ((long long)M * N));
  C[c_grp[g] + c_row[m] + c_col[n]] = s;
}

}  // namespace

cudaError_t launch_igemm_f32(const IGemmLaunch& p, const void* A, const void* B, void* C, const void* const* tables,
                             void* partial, cudaStream_t stream, int* launches) {
  dim3 grid((p.M + BM - 1) / BM, (p.N + BN - 1) / BN, p.groups * p.split_k);
  dim3 block(NT);
  auto a_row = (const RowEnt*)tables[0];
  auto a_col = (const ColEnt*)tables[1];
  auto b_row = (const long long*)tables[2];
  auto b_col = (const long long*)tables[3];
  auto c_row = (const long long*)tables[4];
  auto c_col = (const long long*)tables[5];
  auto a_grp = (const long long*)tables[6];
  auto b_grp = (const long long*)tables[7];
  auto c_grp = (const long long*)tables[8];
#define LAUNCH(AM, BK_, MK)                                                                                          \
  igemm_f32_kernel<AM, BK_, MK><<<grid, block, 0, stream>>>((const float*)A, (const float*)B, (float*)C, a_row, a_col, \
                                                            b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp,           \
                                                            (float*)partial, p)
  int v = (p.a_mcontig ? 4 : 0) | (p.b_kcontig ? 2 : 0) | (p.mask ? 1 : 0);
  switch (v) {
    case 0: LAUNCH(false, false, false); break;
    case 1: LAUNCH(false, false, true); break;
    case 2: LAUNCH(false, true, false); break;
    case 3: LAUNCH(false, true, true); break;
    case 4: LAUNCH(true, false, false); break;
    case 5: LAUNCH(true, false, true); break;
    case 6: LAUNCH(true, true, false); break;
    default: LAUNCH(true, true, true); break;
  }
#undef LAUNCH
  if (launches) (*launches)++;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (p.split_k > 1) {
    long long total = (long long)p.groups * p.M * p.N;
    splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>((const float*)partial, (float*)C, c_row,
                                                                              c_col, c_grp, p.M, p.N, p.groups, p.split_k);
    if (launches) (*launches)++;
    e = cudaGetLastError();
  }
  return e;
}

}  // namespace b200
