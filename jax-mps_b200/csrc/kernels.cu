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
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <algorithm>
#include <mutex>
#include <cstdio>
#include <cstring>

#include "kernels.h"
#include "tc_util.cuh"

namespace b200 {

namespace {
// Launch with programmatic stream serialization (the product kernels and their split-K sum start with pdl_prologue).
bool g_igemm_programmatic_launch = true;

template <typename... P, typename... A>
cudaError_t launch_k(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_igemm_programmatic_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}


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
  pdl_prologue();
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

// Sum of the split-K partial tiles, in a fixed order. Threads (32, KY), or (256, 1) when KY = 1: thread x owns one output (or four consecutive
// n when VEC), row y adds the splits y, y + KY, ... with four independent accumulators so that several loads are in
// flight; the KY rows are then added in order by row 0.
template <int KY, bool VEC>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ partial, float* __restrict__ C,
                                                                const long long* __restrict__ c_row,
                                                                const long long* __restrict__ c_col,
                                                                const long long* __restrict__ c_grp, int M, int N, int groups,
                                                                int split_k) {
  pdl_prologue();
  constexpr int W = VEC ? 4 : 1;
  __shared__ float sm[KY][32 * W + 1];
  const long long total = (long long)groups * M * N;
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * W;     // blockDim.x is 32 when KY > 1
  float acc[4][W];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int w = 0; w < W; ++w) acc[a][w] = 0.f;
  if (i < total) {
    int k = threadIdx.y;
    for (; k + 3 * KY < split_k; k += 4 * KY) {
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float* src = partial + (long long)(k + a * KY) * total + i;
        if (VEC) { const float4 v = *reinterpret_cast<const float4*>(src); acc[a][0] += v.x; acc[a][W > 1 ? 1 : 0] += v.y; acc[a][W > 2 ? 2 : 0] += v.z; acc[a][W > 3 ? 3 : 0] += v.w; }
        else acc[a][0] += *src;
      }
    }
    for (; k < split_k; k += KY) {
      const float* src = partial + (long long)k * total + i;
      if (VEC) { const float4 v = *reinterpret_cast<const float4*>(src); acc[0][0] += v.x; acc[0][W > 1 ? 1 : 0] += v.y; acc[0][W > 2 ? 2 : 0] += v.z; acc[0][W > 3 ? 3 : 0] += v.w; }
      else acc[0][0] += *src;
    }
  }
  float s[W];
#pragma unroll
  for (int w = 0; w < W; ++w) s[w] = (acc[0][w] + acc[1][w]) + (acc[2][w] + acc[3][w]);
  if (KY > 1) {
#pragma unroll
    for (int w = 0; w < W; ++w) sm[threadIdx.y][threadIdx.x * W + w] = s[w];
    __syncthreads();
    if (threadIdx.y != 0) return;
#pragma unroll
    for (int w = 0; w < W; ++w) {
      float t = sm[0][threadIdx.x * W + w];
      for (int y = 1; y < KY; ++y) t += sm[y][threadIdx.x * W + w];
      s[w] = t;
    }
  }
  if (i >= total) return;
  const int n = (int)(i % N);
  const int m = (int)((i / N) % M);
  const int g = (int)(i / ((long long)M * N));
  float* out = C + c_grp[g] + c_row[m] + c_col[n];
  if (VEC) *reinterpret_cast<float4*>(out) = make_float4(s[0], s[W > 1 ? 1 : 0], s[W > 2 ? 2 : 0], s[W > 3 ? 3 : 0]);
  else *out = s[0];
}


// ---------------------------------------------------------------------------
// Tensor-core path: the same table-driven implicit GEMM on tcgen05 (sm_100a).
//
// fp32 operands are split in registers into a TF32-representable high part and
// a low part (x = hi + lo, both rounded to 10 mantissa bits) and the product is
// accumulated as hi*hi + hi*lo + lo*hi by three tcgen05.mma.kind::tf32
// instructions per k-step into one fp32 accumulator in tensor memory: the
// result carries about 21 bits, i.e. fp32-level accuracy, never plain TF32.
//
// One CTA computes a 128 x 64 tile. Per 32-deep k-tile all 256 threads gather
// A (128 x 32) and B (64 x 32) from global memory through the index tables
// (im2col, padding and dilation masks included), split them and store the four
// operand tiles (A hi/lo, B hi/lo) in shared memory in the K-major 128-byte
// swizzled layout the MMA unit reads; one thread then issues 12 MMAs and
// commits them to the stage's mbarrier, so the tensor pipe works on tile k
// while the CTA gathers tile k+1 into the other stage (two CTAs per SM
// interleave further). The accumulator is read back with tcgen05.ld.
// Every mbarrier wait is bounded: on expiry the CTA raises *error_flag, skips
// its stores, releases its tensor memory and returns.
constexpr int TBM = 128, TBN = 64, TBK = 32, TSTAGES = 2, TNT = 256;
constexpr int TA_BYTES = TBM * TBK * 4, TB_BYTES = TBN * TBK * 4;
constexpr int TSTAGE_BYTES = 2 * TA_BYTES + 2 * TB_BYTES;
constexpr int TSMEM_BYTES = TSTAGES * TSTAGE_BYTES + 1024 + 64;

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

// x = hi + lo with hi and lo representable in TF32 (round to nearest on 10 mantissa bits)
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  uint32_t u = __float_as_uint(x);
  uint32_t h = ((u & 0x7F800000u) == 0x7F800000u) ? u : ((u + 0x1000u) & 0xFFFFE000u);
  hi = __uint_as_float(h);
  float l = x - hi;
  uint32_t lu = __float_as_uint(l);
  lo = __uint_as_float(((lu & 0x7F800000u) == 0x7F800000u) ? lu : ((lu + 0x1000u) & 0xFFFFE000u));
}

// byte offset of the 16-byte chunk `chunk` (0..7) of row `r` inside a K-major SW128 tile
__device__ __forceinline__ uint32_t sw128(int r, int chunk) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}

template <bool A_MCONTIG, bool B_KCONTIG, bool MASK>
__global__ void __launch_bounds__(TNT, 2) igemm_tf32x3_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                             float* __restrict__ C, const RowEnt* __restrict__ a_row,
                                                             const ColEnt* __restrict__ a_col,
                                                             const long long* __restrict__ b_row,
                                                             const long long* __restrict__ b_col,
                                                             const long long* __restrict__ c_row,
                                                             const long long* __restrict__ c_col,
                                                             const long long* __restrict__ a_grp,
                                                             const long long* __restrict__ b_grp,
                                                             const long long* __restrict__ c_grp,
                                                             float* __restrict__ partial, int* __restrict__ error_flag,
                                                             IGemmLaunch p) {
  pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = (uint64_t*)(smem + TSTAGES * TSTAGE_BYTES);      // one mbarrier per stage
  uint32_t* tmem_slot = (uint32_t*)(bars + TSTAGES);
  int* failed = (int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * TBM, n0 = blockIdx.y * TBN;
  const int g = blockIdx.z / p.split_k, sp = blockIdx.z % p.split_k;
  const int kchunk = ((p.K + p.split_k - 1) / p.split_k + TBK - 1) / TBK * TBK;
  const int kbeg = sp * kchunk, kend = min(p.K, kbeg + kchunk);
  const int ktiles = kend > kbeg ? (kend - kbeg + TBK - 1) / TBK : 0;
  const float* Ag = A + a_grp[g];
  const float* Bg = B + b_grp[g];

  if (tid == 0) {
    for (int s = 0; s < TSTAGES; ++s) mbar_init(smem_u32(&bars[s]), 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TBN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // ---- what this thread gathers: 4 chunks of A (16 floats) and 2 chunks of B (8 floats) per k-tile ----
  // K-contiguous operand: chunk = tid % 8, rows tid / 8 + 32 i.  M/N-contiguous operand: row = tid % rows, chunks strided.
  RowEnt arow[A_MCONTIG ? 1 : 4];
  bool arow_ok[A_MCONTIG ? 1 : 4];
  if (A_MCONTIG) {
    int m = m0 + (tid & 127);
    arow_ok[0] = m < p.M;
    arow[0] = arow_ok[0] ? a_row[m] : RowEnt{0, 0, 0};
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int m = m0 + (tid >> 3) + 32 * i;
      arow_ok[i] = m < p.M;
      arow[i] = arow_ok[i] ? a_row[m] : RowEnt{0, 0, 0};
    }
  }
  long long bcol[B_KCONTIG ? 2 : 1];
  bool bcol_ok[B_KCONTIG ? 2 : 1];
  if (B_KCONTIG) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int n = n0 + (tid >> 3) + 32 * i;
      bcol_ok[i] = n < p.N;
      bcol[i] = bcol_ok[i] ? b_col[n] : 0;
    }
  } else {
    int n = n0 + (tid & 63);
    bcol_ok[0] = n < p.N;
    bcol[0] = bcol_ok[0] ? b_col[n] : 0;
  }

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

  float ra[16], rb[8];
  auto load_tile = [&](int kt) {
    const int k0 = kbeg + kt * TBK;
    if (A_MCONTIG) {
      // chunks (tid / 128) + 2 j, j = 0..3
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int kq = (tid >> 7) + 2 * j;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int k = k0 + kq * 4 + e;
          bool cok = k < kend;
          ColEnt c = cok ? a_col[k] : ColEnt{0, 0, 0};
          ra[j * 4 + e] = fetch_a(arow[0], arow_ok[0], c, cok);
        }
      }
    } else {
      ColEnt c[4];
      bool cok[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int k = k0 + (tid & 7) * 4 + e;
        cok[e] = k < kend;
        c[e] = cok[e] ? a_col[k] : ColEnt{0, 0, 0};
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) ra[i * 4 + e] = fetch_a(arow[i], arow_ok[i], c[e], cok[e]);
    }
    if (B_KCONTIG) {
      long long br[4];
      bool kok[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        int k = k0 + (tid & 7) * 4 + e;
        kok[e] = k < kend;
        br[e] = kok[e] ? b_row[k] : 0;
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) rb[i * 4 + e] = (kok[e] && bcol_ok[i]) ? __ldg(Bg + br[e] + bcol[i]) : 0.f;
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        int kq = (tid >> 6) + 4 * j;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          int k = k0 + kq * 4 + e;
          bool kok = k < kend;
          rb[j * 4 + e] = (kok && bcol_ok[0]) ? __ldg(Bg + b_row[kok ? k : 0] + bcol[0]) : 0.f;
        }
      }
    }
  };
  auto store_tile = [&](int s) {
    uint8_t* st = smem + s * TSTAGE_BYTES;
    uint8_t *a_hi = st, *a_lo = st + TA_BYTES, *b_hi = st + 2 * TA_BYTES, *b_lo = st + 2 * TA_BYTES + TB_BYTES;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int r = A_MCONTIG ? (tid & 127) : (tid >> 3) + 32 * q;
      int chunk = A_MCONTIG ? (tid >> 7) + 2 * q : (tid & 7);
      float4 h, l;
      split_tf32(ra[q * 4 + 0], h.x, l.x);
      split_tf32(ra[q * 4 + 1], h.y, l.y);
      split_tf32(ra[q * 4 + 2], h.z, l.z);
      split_tf32(ra[q * 4 + 3], h.w, l.w);
      uint32_t off = sw128(r, chunk);
      *reinterpret_cast<float4*>(a_hi + off) = h;
      *reinterpret_cast<float4*>(a_lo + off) = l;
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      int r = B_KCONTIG ? (tid >> 3) + 32 * q : (tid & 63);
      int chunk = B_KCONTIG ? (tid & 7) : (tid >> 6) + 4 * q;
      float4 h, l;
      split_tf32(rb[q * 4 + 0], h.x, l.x);
      split_tf32(rb[q * 4 + 1], h.y, l.y);
      split_tf32(rb[q * 4 + 2], h.z, l.z);
      split_tf32(rb[q * 4 + 3], h.w, l.w);
      uint32_t off = sw128(r, chunk);
      *reinterpret_cast<float4*>(b_hi + off) = h;
      *reinterpret_cast<float4*>(b_lo + off) = l;
    }
  };

  // instruction descriptor: D fp32, A and B tf32, both K-major, N = 64, M = 128
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TBN >> 3) << 17) | ((uint32_t)(TBM >> 4) << 24);
  bool ok = true;
  if (ktiles > 0) load_tile(0);
  for (int kt = 0; kt < ktiles; ++kt) {
    const int s = kt % TSTAGES;
    if (kt >= TSTAGES) {
      // the MMAs that read this stage (k-tile kt - TSTAGES) must have retired
      // (the verdict is made uniform across the CTA so that nobody is left behind at a barrier)
      const bool mine = mbar_wait(smem_u32(&bars[s]), (uint32_t)((kt / TSTAGES - 1) & 1));
      if (!__syncthreads_and(mine)) { ok = false; break; }
    }
    store_tile(s);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy stores -> visible to the MMA unit
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t base = smem_u32(smem + s * TSTAGE_BYTES);
      const uint64_t da_hi = umma_desc(base), da_lo = umma_desc(base + TA_BYTES);
      const uint64_t db_hi = umma_desc(base + 2 * TA_BYTES), db_lo = umma_desc(base + 2 * TA_BYTES + TB_BYTES);
#pragma unroll
      for (int kk = 0; kk < TBK / 8; ++kk) {
        const uint64_t adv = (uint64_t)(kk * 32 >> 4);       // 8 tf32 = 32 bytes along K inside the swizzle atom
        umma_tf32(tmem, da_hi + adv, db_hi + adv, idesc, (kt | kk) != 0);
        umma_tf32(tmem, da_hi + adv, db_lo + adv, idesc, 1);
        umma_tf32(tmem, da_lo + adv, db_hi + adv, idesc, 1);
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[s]))
                   : "memory");
    }
    if (kt + 1 < ktiles) load_tile(kt + 1);
  }
  if (ok && ktiles > 0) {
    const int last = ktiles - 1;
    ok = mbar_wait(smem_u32(&bars[last % TSTAGES]), (uint32_t)((last / TSTAGES) & 1));
  }
  ok = __syncthreads_and(ok);
  if (!ok && tid == 0) {
    *failed = 1;
    atomicAdd(error_flag, 1);
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  // ---- epilogue: warp w reads TMEM lanes 32 (w % 4) .. +31, columns 32 (w / 4) .. +31 ----
  if (ok) {
    uint32_t v[32];
    if (ktiles > 0) {
      const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(32 * (warp >> 2));
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
          "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
            "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
            "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
          : "r"(taddr)
          : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = 0u;
    }
    const int m = m0 + 32 * (warp & 3) + lane;
    const int nb = n0 + 32 * (warp >> 2);
    if (m < p.M) {
      if (p.split_k > 1) {
        float* out = partial + ((long long)sp * p.groups + g) * (long long)p.M * p.N + (long long)m * p.N;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (nb + j < p.N) out[nb + j] = __uint_as_float(v[j]);
      } else {
        float* out = C + c_grp[g] + c_row[m];
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (nb + j < p.N) out[c_col[nb + j]] = __uint_as_float(v[j]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TBN) : "memory");
  }
}


// ---------------------------------------------------------------------------
// Tensor-core path, vector gather: as above, but operands move in 16-byte
// chunks with cp.async (zero-filled where the convolution window falls on
// padding or between dilated input pixels) straight into the swizzled tile the
// MMA unit reads, so the raw fp32 tile is the "high" operand as it stands: the
// tensor core reads only the TF32 bits of each word (sign, exponent, top 10
// mantissa bits). The only transformation is lo = x - trunc_tf32(x), written to
// a second tile. An operand whose contraction index is contiguous in memory is
// stored K-major; one whose row index (m or n) is contiguous is stored
// MN-major, so both kinds gather with full 16-byte requests.
// The host enables this kernel only when every chunk is uniform: four
// consecutive table entries are four consecutive, 16-byte aligned floats
// sharing one window position (IGemmLaunch::vec).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// byte offset of 16-byte chunk `mc` (4 consecutive m or n) at contraction index k (0..31) in an MN-major
// tile. 32-bit operands stored MN-major use the "128-byte swizzle with 32-byte base" layout: atoms of
// 4 k-rows x 128 bytes (32 values along m/n), 32-byte pieces of a row XOR-ed with the row number; atoms are
// ordered k-atom major: offset = (ka * mn_atoms + ma) * 512.
__device__ __forceinline__ uint32_t sw128_mn(int mc, int k, int mn_atoms) {
  const int ma = mc >> 3, c16 = mc & 7, ka = k >> 2, ki = k & 3;
  return (uint32_t)(((ka * mn_atoms + ma) << 9) + (ki << 7) + ((((c16 >> 1) ^ ki)) << 5) + ((c16 & 1) << 4));
}

__device__ __forceinline__ uint64_t umma_desc_mn(uint32_t smem_addr, int mn_atoms) {
  // MN-major, SWIZZLE_128B_BASE32B (layout type 1): LBO = distance between atoms along M/N (512 B),
  // SBO = distance between 4-row atoms along K
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(512 >> 4) << 16) |
         ((uint64_t)((mn_atoms * 512) >> 4) << 32) | (1ull << 46) | (1ull << 61);
}

// ---------------------------------------------------------------------------
// Tensor-core path, warp-specialised (used for every contraction whose operands gather in uniform 16-byte
// chunks). Cycle counters in the roles of earlier versions showed that a handful of warps each walking a long
// dependent chain (table lookup -> mask -> address -> copy; 16 descriptors per k-tile in the MMA thread) bound
// the kernel, not bandwidth or the tensor pipe. Hence many thin roles:
//   warps 0-15, gather : the 16-byte chunks of a k-tile (A then B) form one flat list; thread t takes chunks
//       t, t + 512, ...; each is one table lookup pair, one mask test and one cp.async (zero-filled where the
//       window falls on padding or a dilation hole) into the raw tile of a ring stage; the thread's copies
//       arrive on the stage's `landed` barrier when they complete. The warps run up to STAGES - 1 tiles ahead.
//   warps 16-23, low part: wait for `landed`, read chunks back, store lo = x - tf32(x) into the stage's
//       low-part tile, fence towards the async proxy and arrive on `ready`.
//   warp 24, one thread : waits for `ready`, issues the 12 MMAs of the tile (raw x raw, raw x lo, lo x raw per
//       k-step) from descriptors prepared before the loop, commits them to the stage's `empty` barrier.
// After the last commit warps 0-7 read the accumulator from tensor memory and store it.
// All waits are bounded; a role that times out raises the error word and leaves its loop, the others time
// out in turn, everybody meets at the final barrier and tensor memory is released.
template <int BN_>
struct WsCfg {
  static constexpr int BN = BN_;
  static constexpr int STAGES = BN_ == 64 ? 4 : 3;
  static constexpr int A_BYTES = TBM * TBK * 4, B_BYTES = BN_ * TBK * 4;
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);          // raw A, raw B, low A, low B
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 512;
  static constexpr int A_CHUNKS = TBM * TBK / 4, B_CHUNKS = BN_ * TBK / 4;
};
// role sizes: chunk gather 512 + 256 low-part threads, segment gather 256 + 512; one more warp issues the MMAs
constexpr int WS_THREADS = 768 + 32;

// Accumulator read-back shared by the tensor-core kernels: eight warps; warp `ew` reads TMEM lanes 32 * (ew & 3) ..
// (row m0 + lane of that quadrant) and the column half ew >> 2, waits (bounded) for the MMAs of the last k-tile
// (barrier `last_bar`, phase `last_parity`), and stores to C or to the split-K partial buffer.
template <int BN>
__device__ __forceinline__ void store_accumulator(uint32_t tmem, int warp, int lane, int m0, int n0, int g, int sp, int ktiles,
                                                  const IGemmLaunch& p, float* __restrict__ C, float* __restrict__ partial,
                                                  const long long* __restrict__ c_row, const long long* __restrict__ c_col,
                                                  const long long* __restrict__ c_grp, volatile int* failed,
                                                  uint32_t last_bar, uint32_t last_parity) {
  bool ok = !*failed;
  if (ok && ktiles > 0) {
    ok = mbar_wait(last_bar, last_parity);
    if (!ok) *failed = 1;
  }
  ok = __all_sync(0xFFFFFFFFu, ok);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
    const int m = m0 + 32 * (warp & 3) + lane;
#pragma unroll
    for (int part = 0; part < BN / 64; ++part) {
      const int col0 = (warp >> 2) * (BN / 2) + part * 32;
      uint32_t v[32];
      if (ktiles > 0) {
        const uint32_t taddr = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)col0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
            "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
              "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
              "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
              "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int q = 0; q < 32; ++q) v[q] = 0u;
      }
      const int nb = n0 + col0;
      if (m < p.M && nb < p.N) {
        float* out;
        bool contiguous;
        if (p.split_k > 1) {
          out = partial + ((long long)sp * p.groups + g) * (long long)p.M * p.N + (long long)m * p.N + nb;
          contiguous = (p.N & 3) == 0;
        } else {
          out = C + c_grp[g] + c_row[m] + c_col[nb];
          contiguous = p.c_vec != 0;
        }
        if (contiguous && nb + 32 <= p.N && (((uintptr_t)out) & 15) == 0) {
#pragma unroll
          for (int q = 0; q < 32; q += 4)
            *reinterpret_cast<float4*>(out + q) = make_float4(__uint_as_float(v[q]), __uint_as_float(v[q + 1]),
                                                              __uint_as_float(v[q + 2]), __uint_as_float(v[q + 3]));
        } else if (p.split_k > 1) {
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (nb + q < p.N) out[q] = __uint_as_float(v[q]);
        } else {
          float* row = C + c_grp[g] + c_row[m];
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (nb + q < p.N) row[c_col[nb + q]] = __uint_as_float(v[q]);
        }
      }
    }
  }
}

template <int BN, bool A_MCONTIG, bool B_KCONTIG, bool MASK, bool SEG>
__global__ void __launch_bounds__(WS_THREADS, 1) igemm_tf32x3_ws_kernel(
    const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, const RowEnt* __restrict__ a_row,
    const ColEnt* __restrict__ a_col, const long long* __restrict__ b_row, const long long* __restrict__ b_col,
    const long long* __restrict__ c_row, const long long* __restrict__ c_col, const long long* __restrict__ a_grp,
    const long long* __restrict__ b_grp, const long long* __restrict__ c_grp, float* __restrict__ partial,
    int* __restrict__ error_flag, IGemmLaunch p) {
  pdl_prologue();
  using Cfg = WsCfg<BN>;
  constexpr int S = Cfg::STAGES;
  constexpr int WS_GATHER = SEG ? 256 : 512, WS_LOW = 768 - WS_GATHER;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* landed = (uint64_t*)(smem + S * Cfg::STAGE_BYTES);
  uint64_t* ready = landed + S;
  uint64_t* empty = ready + S;
  uint64_t* done = empty + S;                      // completes once, when every MMA of the CTA has retired
  uint32_t* tmem_slot = (uint32_t*)(done + 1);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * TBM, n0 = blockIdx.y * BN;
  const int g = blockIdx.z / p.split_k, sp = blockIdx.z % p.split_k;
  const int kchunk = ((p.K + p.split_k - 1) / p.split_k + TBK - 1) / TBK * TBK;
  const int kbeg = sp * kchunk, kend = min(p.K, kbeg + kchunk);
  const int ktiles = kend > kbeg ? (kend - kbeg + TBK - 1) / TBK : 0;
  constexpr int MMA_WARP = (WS_GATHER + WS_LOW) / 32;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&landed[s]), WS_GATHER);
      mbar_init(smem_u32(&ready[s]), WS_LOW);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(done), 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // flat chunk index -> (offset inside the A or B tile, row index, k index of the chunk's first element)
  //   K-major tile : chunk = row * 8 + kc         (4 consecutive k of one row)
  //   MN-major tile: chunk = k * (rows / 4) + rc  (4 consecutive rows at one k)
  auto a_chunk = [&](int idx, int& row, int& k) -> uint32_t {
    if (A_MCONTIG) { k = idx >> 5; row = (idx & 31) * 4; return sw128_mn(idx & 31, k, TBM / 32); }
    row = idx >> 3; k = (idx & 7) * 4; return sw128(row, idx & 7);
  };
  auto b_chunk = [&](int idx, int& row, int& k) -> uint32_t {
    if (B_KCONTIG) { row = idx >> 3; k = (idx & 7) * 4; return sw128(row, idx & 7); }
    constexpr int BMC = BN / 4;
    k = idx / BMC; row = (idx % BMC) * 4; return sw128_mn(idx % BMC, k, BN / 32);
  };

  if (SEG && tid < WS_GATHER) {
    // ------------------------------ gather by 128-byte rows --------------------------------------------------
    // The host sets IGemmLaunch::seg when every aligned run of 32 indices along an operand's contiguous
    // dimension is 32 consecutive floats sharing one window position. A row of the swizzled tile (K-major:
    // one m or n with 32 k; MN-major: one k with 32 m or n) is then one 128-byte line of memory with one
    // address and one padding mask. Warps 0-3 own 32 rows of the A tile each, warps 4-7 own BN / 4 rows of
    // the B tile each: lane l works out address and mask of row l, then the warp copies four rows per
    // instruction, eight lanes per row, so every cp.async instruction touches four whole lines.
    const int a_sh = (int)p.a_sh, a_sw = (int)p.a_sw;
    const bool is_a = warp < 4;
    constexpr int B_ROWS = BN / 4;                   // rows per B warp
    const int rows = is_a ? 32 : B_ROWS;
    const int u = is_a ? warp * 32 + lane : (warp - 4) * B_ROWS + (lane % B_ROWS);   // tile row owned by this lane
    int k_local = 0;                                 // MN-major rows sit at their own k inside the tile
    uint32_t x_off;                                  // byte offset of the row in the stage, swizzle key folded in
    int base_off = -1, h0 = 0, w0 = 0;               // m- or n-dependent part of the address (-1: out of range)
    const float* src_base;
    if (is_a) {
      src_base = A + a_grp[g];
      int m;
      if (A_MCONTIG) { k_local = u >> 2; const int mg = u & 3; m = m0 + mg * 32;
        x_off = (uint32_t)((((k_local >> 2) * (TBM / 32) + mg) << 9) + ((k_local & 3) << 7) + ((k_local & 3) << 5));
      } else { m = m0 + u; x_off = (uint32_t)((u >> 3) * 1024 + (u & 7) * 128 + ((u & 7) << 4)); }
      if (m < p.M) { const RowEnt r = a_row[m]; base_off = (int)r.off; h0 = r.h0; w0 = r.w0; }
    } else {
      src_base = B + b_grp[g];
      int n;
      if (B_KCONTIG) { n = n0 + u; x_off = (uint32_t)((u >> 3) * 1024 + (u & 7) * 128 + ((u & 7) << 4)); }
      else { k_local = u / (BN / 32); const int ng = u % (BN / 32); n = n0 + ng * 32;
        x_off = (uint32_t)((((k_local >> 2) * (BN / 32) + ng) << 9) + ((k_local & 3) << 7) + ((k_local & 3) << 5)); }
      if (n < p.N) base_off = (int)b_col[n];
      x_off += Cfg::A_BYTES;
    }
    // destination of this lane's chunk in the q-th group of four rows
    const int cl = lane & 7;
    uint32_t dst[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) dst[q] = __shfl_sync(0xFFFFFFFFu, x_off, (4 * q + (lane >> 3)) % rows) ^ (uint32_t)(cl << 4);
    src_base += 4 * cl;
    struct Ent { int off, dh, dw; };
    // k-dependent table entry of tile j for this lane's row; fetched two tiles ahead into alternating registers
    auto fetch = [&](int j, Ent& e) {
      const int k = kbeg + j * TBK + k_local;
      e.off = -1; e.dh = 0; e.dw = 0;
      if (j < ktiles && k < kend) {
        if (is_a) { const ColEnt c = a_col[k]; e.off = (int)c.off; e.dh = c.dh; e.dw = c.dw; }
        else e.off = (int)b_row[k];
      }
    };
    auto tile = [&](int j, const Ent& e) -> bool {
      const int s = j % S;
      bool valid = base_off >= 0 && e.off >= 0;
      int o = base_off + e.off;
      if (MASK && is_a) {
        int ih = h0 + e.dh, iw = w0 + e.dw;
        valid = valid && ih >= 0 && iw >= 0 && ih < p.Hd && iw < p.Wd;
        if (p.ldh != 1) { valid = valid && (ih % p.ldh == 0); ih /= p.ldh; }
        if (p.ldw != 1) { valid = valid && (iw % p.ldw == 0); iw /= p.ldw; }
        o += ih * a_sh + iw * a_sw;
      }
      if (!valid) o = -1;
      if (j >= S) {
        // the MMAs of tile j - S were the last readers of this stage
        // the warp leaves together: the shuffles below name every lane
        if (!__all_sync(0xFFFFFFFFu, !*failed && mbar_wait(smem_u32(&empty[s]), (uint32_t)((j / S - 1) & 1)))) { *failed = 1; return false; }
      }
      const uint32_t x = smem_u32(smem + s * Cfg::STAGE_BYTES);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (4 * q < rows) {
          const int oq = __shfl_sync(0xFFFFFFFFu, o, 4 * q + (lane >> 3));
          cp_async16(x + dst[q], oq >= 0 ? src_base + oq : src_base, oq >= 0);
        }
      }
      // this thread's arrival on `landed` fires when its copies above have completed
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&landed[s])) : "memory");
      return true;
    };
    Ent e0, e1;
    fetch(0, e0);
    fetch(1, e1);
    for (int j = 0; j < ktiles; j += 2) {
      if (!tile(j, e0)) break;
      fetch(j + 2, e0);
      if (j + 1 < ktiles) {
        if (!tile(j + 1, e1)) break;
        fetch(j + 3, e1);
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (!SEG && tid < WS_GATHER) {
    // ------------------------------ gather -----------------------------------------------------------------
    const float* Ag = A + a_grp[g];
    const float* Bg = B + b_grp[g];
    const int a_sh = (int)p.a_sh, a_sw = (int)p.a_sw;
    // A thread's chunks sit at the same rows and k offsets in every k-tile: row lookups happen once, here;
    // per tile only the k-dependent entries are fetched.
    constexpr int NA = Cfg::A_CHUNKS / WS_GATHER, NBQ = Cfg::B_CHUNKS / WS_GATHER;
    uint32_t a_so[NA], b_so[NBQ];
    int a_kk[NA], b_kk[NBQ], a_ro[NA], a_h0[NA], a_w0[NA], b_no[NBQ];
#pragma unroll
    for (int q = 0; q < NA; ++q) {
      int row;
      a_so[q] = a_chunk(tid + q * WS_GATHER, row, a_kk[q]);
      const int m = m0 + row;
      if (m < p.M) { const RowEnt r = a_row[m]; a_ro[q] = (int)r.off; a_h0[q] = r.h0; a_w0[q] = r.w0; }
      else { a_ro[q] = -1; a_h0[q] = 0; a_w0[q] = 0; }
    }
#pragma unroll
    for (int q = 0; q < NBQ; ++q) {
      int row;
      b_so[q] = b_chunk(tid + q * WS_GATHER, row, b_kk[q]);
      const int n = n0 + row;
      b_no[q] = n < p.N ? (int)b_col[n] : -1;
    }
    for (int j = 0; j < ktiles; ++j) {
      const int s = j % S;
      const int k0 = kbeg + j * TBK;
      // k-dependent table entries first: their latency overlaps the wait for the stage
      ColEnt ac[NA];
      int br[NBQ];
#pragma unroll
      for (int q = 0; q < NA; ++q) {
        const int k = k0 + a_kk[q];
        ac[q] = (k < kend && (q == 0 || A_MCONTIG)) ? a_col[k] : ColEnt{-1, 0, 0};
        if (!A_MCONTIG && q > 0) ac[q] = ac[0];                 // K-major: all of a thread's chunks share one k
        if (k >= kend) ac[q].off = -1;
      }
#pragma unroll
      for (int q = 0; q < NBQ; ++q) {
        const int k = k0 + b_kk[q];
        br[q] = k < kend ? (int)b_row[k] : -1;
      }
      if (j >= S) {
        // the MMAs of tile j - S were the last readers of this stage
        if (*failed || !mbar_wait(smem_u32(&empty[s]), (uint32_t)((j / S - 1) & 1))) { *failed = 1; break; }
      }
      const uint32_t a_raw = smem_u32(smem + s * Cfg::STAGE_BYTES), b_raw = a_raw + Cfg::A_BYTES;
#pragma unroll
      for (int q = 0; q < NA; ++q) {
        bool valid = a_ro[q] >= 0 && ac[q].off >= 0;
        int o = a_ro[q] + (int)ac[q].off;
        if (MASK) {
          int ih = a_h0[q] + ac[q].dh, iw = a_w0[q] + ac[q].dw;
          valid = valid && ih >= 0 && iw >= 0 && ih < p.Hd && iw < p.Wd;
          if (p.ldh != 1) { valid = valid && (ih % p.ldh == 0); ih /= p.ldh; }
          if (p.ldw != 1) { valid = valid && (iw % p.ldw == 0); iw /= p.ldw; }
          o += ih * a_sh + iw * a_sw;
        }
        cp_async16(a_raw + a_so[q], valid ? Ag + o : Ag, valid);
      }
#pragma unroll
      for (int q = 0; q < NBQ; ++q) {
        const bool valid = b_no[q] >= 0 && br[q] >= 0;
        cp_async16(b_raw + b_so[q], valid ? Bg + br[q] + b_no[q] : Bg, valid);
      }
      // this thread's arrival on `landed` fires when its copies above have completed
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&landed[s])) : "memory");
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (tid < WS_GATHER + WS_LOW) {
    // ------------------------------ low part ----------------------------------------------------------------
    const int t = tid - WS_GATHER;
    // lo = x - (TF32 bits of x): exact in fp32. Adding half a TF32 unit to its bit pattern makes the tensor
    // core's truncation of the stored word a round-to-nearest. An infinite x would give inf - inf = NaN; those
    // are rare, so the fast pass only tracks max|x| and a tile that saw an infinity is redone element-wise.
    auto lo1 = [](float x) -> float {
      const float l = x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
      return __uint_as_float(__float_as_uint(l) + 0x1000u);
    };
    auto lo1_safe = [&](float x) -> float { return fabsf(x) == INFINITY ? 0.f : lo1(x); };
    for (int j = 0; j < ktiles; ++j) {
      const int s = j % S;
      if (*failed || !mbar_wait(smem_u32(&landed[s]), (uint32_t)((j / S) & 1))) { *failed = 1; break; }
      uint8_t* raw = smem + s * Cfg::STAGE_BYTES;                 // raw A, raw B contiguous; low parts follow
      uint8_t* low = raw + Cfg::A_BYTES + Cfg::B_BYTES;
      // the swizzle only permutes 16-byte chunks inside a tile, so the low-part pass can walk the bytes linearly
      constexpr int NQ = (Cfg::A_CHUNKS + Cfg::B_CHUNKS) / WS_LOW;
      float mx = 0.f;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const uint32_t off = (uint32_t)(t + q * WS_LOW) * 16u;
        const float4 v = *reinterpret_cast<const float4*>(raw + off);
        mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        *reinterpret_cast<float4*>(low + off) = make_float4(lo1(v.x), lo1(v.y), lo1(v.z), lo1(v.w));
      }
      if (mx == INFINITY) {
        for (int q = 0; q < NQ; ++q) {
          const uint32_t off = (uint32_t)(t + q * WS_LOW) * 16u;
          const float4 v = *reinterpret_cast<const float4*>(raw + off);
          *reinterpret_cast<float4*>(low + off) = make_float4(lo1_safe(v.x), lo1_safe(v.y), lo1_safe(v.z), lo1_safe(v.w));
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(smem_u32(&ready[s]));
    }
  } else {
    // ------------------------------ MMA issuer (whole warp, one elected lane issues) --------------------------
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_MCONTIG ? 1u : 0u) << 15) |
                           ((B_KCONTIG ? 0u : 1u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TBM >> 4) << 24);
    // descriptors of stage 0; another stage adds STAGE_BYTES / 16 to the address field, a k-step adds a constant
    const uint32_t base0 = smem_u32(smem);
    const uint64_t d_a = A_MCONTIG ? umma_desc_mn(base0, TBM / 32) : umma_desc(base0);
    const uint64_t d_b = B_KCONTIG ? umma_desc(base0 + Cfg::A_BYTES) : umma_desc_mn(base0 + Cfg::A_BYTES, BN / 32);
    constexpr uint64_t LOW = (uint64_t)((Cfg::A_BYTES + Cfg::B_BYTES) >> 4);
    constexpr uint64_t A_STEP = (uint64_t)((A_MCONTIG ? (TBM / 32) * 1024 : 32) >> 4);
    constexpr uint64_t B_STEP = (uint64_t)((B_KCONTIG ? 32 : (BN / 32) * 1024) >> 4);
    for (int j = 0; j < ktiles; ++j) {
      const int s = j % S;
      const bool ok = !*failed && mbar_wait(smem_u32(&ready[s]), (uint32_t)((j / S) & 1));
      if (!__all_sync(0xFFFFFFFFu, ok)) { *failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t st = (uint64_t)((s * Cfg::STAGE_BYTES) >> 4);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < TBK / 8; ++kk) {
          const uint64_t da = d_a + st + kk * A_STEP, db = d_b + st + kk * B_STEP;
          umma_tf32(tmem, da, db, idesc, (j | kk) != 0);
          umma_tf32(tmem, da, db + LOW, idesc, 1);
          umma_tf32(tmem, da + LOW, db, idesc, 1);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[s]))
                     : "memory");
      }
      __syncwarp();
    }
    // the read-back warps may be several k-tiles ahead of the MMAs, so they wait on a barrier of its own that a
    // last commit completes exactly once (a parity wait on a stage barrier is only unambiguous within one phase)
    if (elect_one())
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done)) : "memory");
    __syncwarp();
  }

  if (warp < 8)
    store_accumulator<BN>(tmem, warp, lane, m0, n0, g, sp, ktiles, p, C, partial, c_row, c_col, c_grp, failed,
                          smem_u32(done), 0u);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *failed) atomicAdd(error_flag, 1);
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Tensor-core path with the A operand in tensor memory (used when both operands gather by whole 128-byte rows,
// IGemmLaunch::seg). Timelines of the kernel above showed it bound by shared-memory traffic: per 32-deep k-tile
// the MMA unit read 72 KB of operands (A three times, B three times) next to 72 KB of copies and low-part
// passes. Here only B lives in shared memory as an MMA operand. A goes global -> shared (raw, cp.async) ->
// registers of one thread per row -> tensor memory, as a high tile (the raw words: the tensor core reads their
// TF32 bits) and a low tile (x - tf32(x)), and tcgen05.mma takes it from there; per k-tile the shared memory
// moves 16 KB + 16 KB for A and (8 + 16 + 24) KB for a 64-wide B instead of 144 KB.
// Roles (warp ranges for the 64-wide tile | the 128-wide tile | the half-size CTA):
//   gather A    0-7 | 0-7 | 0-3    groups of four warps alternating k-tiles (one group in the half-size CTA): lane l owns
//               row l of the warp's 32 tile rows (address + padding mask once per row and k-tile), copies go out four
//               rows per instruction, eight lanes per row (128-byte cp.async.bulk row copies were tried: 1.6x slower)
//   gather B    8-11 | 8-11 | 4-5  the same way, every k-tile
//   convert A   12-19 | 12-15 | 6-9  groups of four warps (two groups alternating k-tiles for the 64-wide tile): thread
//               = one row m of the tile; reads its 32 values (K-major rows: eight 16-byte reads from the swizzled row;
//               MN-major: 32 words, one per k), tcgen05.st of the high and the low words into the stage's 64
//               tensor-memory columns; the same warps read the accumulator back at the end
//   low part B  20-23 | 16-23 | 10-11  in shared memory
// Every producer warp needs about a thousand cycles per k-tile whatever its share of the work (dependent chains), so
// the split gives each role as many independent chains as its share of the critical path needs; the numbers above
// are the fastest of the splits measured.
//   last warp   one thread issues the 12 MMAs of a k-tile (A hi x B raw, A hi x B lo, A lo x B raw per k-step)
//               and commits them to the stage's `empty` barrier
// Tensor memory: all 512 columns; accumulator in [0, BN), A ring from column 128 (64 columns per stage).
// Every wait is bounded as in the kernels above.
// HALF: a CTA of 13 warps with three stages and 256 tensor-memory columns, two of which share an SM, so that the
// launch, pipeline fill and read-back of one overlap the main loop of the other (used for 64-wide tiles when the
// grid has several waves of CTAs).
template <int BN_, bool HALF>
struct TaCfg {
  static constexpr int BN = BN_;
  static constexpr int STAGES = HALF ? 3 : (BN_ == 64 ? 6 : 4);
  static constexpr int A_BYTES = TBM * TBK * 4, B_BYTES = BN_ * TBK * 4;
  static constexpr int STAGE_BYTES = A_BYTES + 2 * B_BYTES;            // raw A, raw B, low B
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 512;
  static constexpr int B_CHUNKS = BN_ * TBK / 4;
  static constexpr int TMEM_COLS = HALF ? 256 : 512;
  static constexpr int A_COL0 = HALF ? 64 : 128;                       // 64 columns per stage after the accumulator
  static constexpr int THREADS = HALF ? 416 : 800;
};

__device__ __forceinline__ void umma_tf32_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, "
      "%25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}

template <int BN, bool A_MCONTIG, bool B_KCONTIG, bool MASK, bool HALF>
__global__ void __launch_bounds__((TaCfg<BN, HALF>::THREADS), (HALF ? 2 : 1)) igemm_tf32x3_ta_kernel(
    const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, const RowEnt* __restrict__ a_row,
    const ColEnt* __restrict__ a_col, const long long* __restrict__ b_row, const long long* __restrict__ b_col,
    const long long* __restrict__ c_row, const long long* __restrict__ c_col, const long long* __restrict__ a_grp,
    const long long* __restrict__ b_grp, const long long* __restrict__ c_grp, float* __restrict__ partial,
    const int* __restrict__ kt_table, int* __restrict__ error_flag, const __grid_constant__ CUtensorMap tm_a, IGemmLaunch p) {
  pdl_prologue();
  using Cfg = TaCfg<BN, HALF>;
  constexpr int S = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* landed_a = (uint64_t*)(smem + S * Cfg::STAGE_BYTES);
  uint64_t* landed_b = landed_a + S;
  uint64_t* a_ready = landed_b + S;
  uint64_t* b_ready = a_ready + S;
  uint64_t* empty = b_ready + S;
  uint64_t* done = empty + S;                      // completes once, when every MMA of the CTA has retired
  uint32_t* tmem_slot = (uint32_t*)(done + 1);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.x * TBM, n0 = blockIdx.y * BN;
  const int g = blockIdx.z / p.split_k, sp = blockIdx.z % p.split_k;
  const int kchunk = ((p.K + p.split_k - 1) / p.split_k + TBK - 1) / TBK * TBK;
  const int kbeg = sp * kchunk, kend = min(p.K, kbeg + kchunk);
  // with a k-tile list (input-dilated convolutions: most window positions of a row tile fall on holes) only the
  // listed k-tiles are visited; j below counts visited tiles, kt_of(j) is the k-tile itself
  const int* kt_list = kt_table ? kt_table + (size_t)blockIdx.x * (p.kt_stride + 1) : nullptr;
  const int ktiles = kt_list ? kt_list[0] : (kend > kbeg ? (kend - kbeg + TBK - 1) / TBK : 0);
  auto kt_of = [&](int j) { return kt_list ? kt_list[1 + j] : j; };
  constexpr int MMA_WARP = Cfg::THREADS / 32 - 1;
  // warp roles in order: A gather groups, B gather, A converter groups, low part of B (the warps that remain), MMA
  constexpr int A_GROUPS = HALF ? 1 : 2;
  constexpr int NBW = HALF ? 2 : 4;                  // B gather warps
  constexpr int CONV_GROUPS = (HALF || BN == 128) ? 1 : 2;          // groups of four converter warps
  constexpr int W_B = 4 * A_GROUPS, W_CONV = W_B + NBW, W_LOW = W_CONV + 4 * CONV_GROUPS, N_LOW = (MMA_WARP - W_LOW) * 32;

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&landed_a[s]), p.a_tma ? 1 : 128);      // one arrival that announces the copy's bytes, or 128 gather threads
      mbar_init(smem_u32(&landed_b[s]), NBW * 32);
      mbar_init(smem_u32(&a_ready[s]), 128);
      mbar_init(smem_u32(&b_ready[s]), N_LOW);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    mbar_init(smem_u32(done), 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  // lo = x - (TF32 bits of x), exact in fp32; adding half a TF32 unit to its bit pattern turns the tensor core's
  // truncation of the stored word into round-to-nearest. inf - inf would be NaN: callers track max|x| and redo
  // a row or tile that saw an infinity with lo1_safe.
  auto lo1 = [](float x) -> float {
    const float l = x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    return __uint_as_float(__float_as_uint(l) + 0x1000u);
  };
  auto lo1_safe = [&](float x) -> float { return fabsf(x) == INFINITY ? 0.f : lo1(x); };

  if (p.a_tma && warp < W_B) {
    // ------------------------------ A by TMA ------------------------------------------------------------------
    // A stride-1 convolution over a dense NHWC input: the 128 rows of this tile are whole output rows, so the A tile
    // of a k-tile (32 channels at one filter tap) is one box of the input, 32 channels x OW pixels x rows x images,
    // and arrives by a single tiled copy in the swizzled row layout the converter threads read; taps that reach
    // outside the image read zeros. One lane of the first warp issues the copies; the other gather warps rest.
    if (warp == 0) {
      const int pixels = p.tma_oh * p.tma_ow;
      const int n0 = m0 / pixels, oh0 = (m0 % pixels) / p.tma_ow;
      const int c_tiles = p.tma_c / TBK;
      for (int j = 0; j < ktiles; ++j) {
        const int s = j % S;
        bool ok = true;
        if (j >= S) ok = !*failed && mbar_wait(smem_u32(&empty[s]), (uint32_t)((j / S - 1) & 1));
        if (!__all_sync(0xFFFFFFFFu, ok)) { *failed = 1; break; }
        if (elect_one()) {
          const int kt = kbeg / TBK + j;
          const int tap = kt / c_tiles, c0 = (kt - tap * c_tiles) * TBK;
          const int kh = tap / p.tma_kw, kw = tap - kh * p.tma_kw;
          const uint32_t bar = smem_u32(&landed_a[s]);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)Cfg::A_BYTES) : "memory");
          asm volatile(
              "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
              ::"r"(smem_u32(smem + s * Cfg::STAGE_BYTES)), "l"(&tm_a), "r"(bar), "r"(c0), "r"(kw * p.tma_rdil_w - p.tma_pad_w),
                "r"(oh0 + kh * p.tma_rdil_h - p.tma_pad_h), "r"(n0)
              : "memory");
        }
        __syncwarp();
      }
    }
  } else if (warp < W_CONV) {
    // ------------------------------ gather -----------------------------------------------------------------
    // A groups take the A tiles of k-tiles group, group + A_GROUPS, ...; the B warps take every B tile
    const int a_sh = (int)p.a_sh, a_sw = (int)p.a_sw;
    const bool is_a = warp < W_B;
    const int first = is_a ? (warp >> 2) : 0, stride = is_a ? A_GROUPS : 1;     // k-tiles first, first + stride, ...
    constexpr int B_ROWS = BN / NBW;                 // rows per B warp
    const int rows = is_a ? 32 : B_ROWS;
    const int u = is_a ? (warp & 3) * 32 + lane : (warp - W_B) * B_ROWS + (lane % B_ROWS);   // tile row owned by this lane
    int k_local = 0;                                 // MN-major rows sit at their own k inside the tile
    uint32_t x_off;                                  // byte offset of the row in the stage (swizzle key folded in)
    int base_off = -1, h0 = 0, w0 = 0;               // m- or n-dependent part of the address (-1: out of range)
    const float* src_base;
    if (is_a) {
      src_base = A + a_grp[g];
      int m;
      // the raw A tile is only read by the converter threads: MN-major rows are stored plainly as [k][128 m],
      // K-major rows as [m][32 k] with the 16-byte chunks XOR-ed by the row number (conflict-free row reads)
      if (A_MCONTIG) { k_local = u >> 2; const int mg = u & 3; m = m0 + mg * 32; x_off = (uint32_t)(k_local * 512 + mg * 128); }
      else { m = m0 + u; x_off = (uint32_t)(u * 128 + ((u & 7) << 4)); }
      if (m < p.M) { const RowEnt r = a_row[m]; base_off = (int)r.off; h0 = r.h0; w0 = r.w0; }
    } else {
      src_base = B + b_grp[g];
      int n;
      if (B_KCONTIG) { n = n0 + u; x_off = (uint32_t)((u >> 3) * 1024 + (u & 7) * 128 + ((u & 7) << 4)); }
      else { k_local = u / (BN / 32); const int ng = u % (BN / 32); n = n0 + ng * 32;
        x_off = (uint32_t)((((k_local >> 2) * (BN / 32) + ng) << 9) + ((k_local & 3) << 7) + ((k_local & 3) << 5)); }
      if (n < p.N) base_off = (int)b_col[n];
      x_off += Cfg::A_BYTES;
    }
    const int cl = lane & 7;
    uint32_t dst[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) dst[q] = __shfl_sync(0xFFFFFFFFu, x_off, (4 * q + (lane >> 3)) % rows) ^ (uint32_t)(cl << 4);
    src_base += 4 * cl;
    uint64_t* landed = is_a ? landed_a : landed_b;
    struct Ent { int off, dh, dw; };
    // k-dependent table entry of tile j for this lane's row, fetched two tiles ahead into alternating registers
    auto fetch = [&](int j, Ent& e) {
      e.off = -1; e.dh = 0; e.dw = 0;
      const int k = j < ktiles ? kbeg + kt_of(j) * TBK + k_local : kend;
      if (j < ktiles && k < kend) {
        if (is_a) { const ColEnt c = a_col[k]; e.off = (int)c.off; e.dh = c.dh; e.dw = c.dw; }
        else e.off = (int)b_row[k];
      }
    };
    auto tile = [&](int j, const Ent& e) -> bool {
      const int s = j % S;
      bool valid = base_off >= 0 && e.off >= 0;
      int o = base_off + e.off;
      if (MASK && is_a) {
        int ih = h0 + e.dh, iw = w0 + e.dw;
        valid = valid && ih >= 0 && iw >= 0 && ih < p.Hd && iw < p.Wd;
        if (p.ldh != 1) { valid = valid && (ih % p.ldh == 0); ih /= p.ldh; }
        if (p.ldw != 1) { valid = valid && (iw % p.ldw == 0); iw /= p.ldw; }
        o += ih * a_sh + iw * a_sw;
      }
      if (!valid) o = -1;
      if (j >= S) {
        // the MMAs of tile j - S were the last readers of this stage (shared memory and tensor memory)
        // the warp leaves together: the shuffles below name every lane
        if (!__all_sync(0xFFFFFFFFu, !*failed && mbar_wait(smem_u32(&empty[s]), (uint32_t)((j / S - 1) & 1)))) { *failed = 1; return false; }
      }
      const uint32_t x = smem_u32(smem + s * Cfg::STAGE_BYTES);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        if (4 * q < rows) {
          const int oq = __shfl_sync(0xFFFFFFFFu, o, 4 * q + (lane >> 3));
          cp_async16(x + dst[q], oq >= 0 ? src_base + oq : src_base, oq >= 0);
        }
      }
      // this thread's arrival on the barrier fires when its copies above have completed
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&landed[s])) : "memory");
      return true;
    };
    Ent e0, e1;
    fetch(first, e0);
    fetch(first + stride, e1);
    for (int j = first; j < ktiles; j += 2 * stride) {
      if (!tile(j, e0)) break;
      fetch(j + 2 * stride, e0);
      if (j + stride < ktiles) {
        if (!tile(j + stride, e1)) break;
        fetch(j + 3 * stride, e1);
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp < W_LOW) {
    // ------------------------------ A: shared memory -> registers -> tensor memory ---------------------------
    const int grp = (warp - W_CONV) >> 2, quad = warp & 3;
    const int row = 32 * quad + lane;
    for (int j = grp; j < ktiles; j += CONV_GROUPS) {
      const int s = j % S;
      if (*failed || !mbar_wait(smem_u32(&landed_a[s]), (uint32_t)((j / S) & 1))) { *failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint8_t* raw = smem + s * Cfg::STAGE_BYTES;
      uint32_t v[32];
      if (A_MCONTIG) {
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = *reinterpret_cast<const uint32_t*>(raw + k * 512 + row * 4);
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 t = *reinterpret_cast<const uint4*>(raw + row * 128 + ((c ^ (row & 7)) << 4));
          v[4 * c] = t.x; v[4 * c + 1] = t.y; v[4 * c + 2] = t.z; v[4 * c + 3] = t.w;
        }
      }
      const uint32_t taddr = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(Cfg::A_COL0 + s * 64);
      tmem_store32(taddr, v);
      float mx = 0.f;
#pragma unroll
      for (int k = 0; k < 32; ++k) mx = fmaxf(mx, fabsf(__uint_as_float(v[k])));
      if (mx == INFINITY) {
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(lo1_safe(__uint_as_float(v[k])));
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = __float_as_uint(lo1(__uint_as_float(v[k])));
      }
      tmem_store32(taddr + 32, v);
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(smem_u32(&a_ready[s]));
    }
  } else if (warp < MMA_WARP) {
    // ------------------------------ low part of B ------------------------------------------------------------
    const int t = tid - W_LOW * 32;
    for (int j = 0; j < ktiles; ++j) {
      const int s = j % S;
      if (*failed || !mbar_wait(smem_u32(&landed_b[s]), (uint32_t)((j / S) & 1))) { *failed = 1; break; }
      uint8_t* raw = smem + s * Cfg::STAGE_BYTES + Cfg::A_BYTES;
      uint8_t* low = raw + Cfg::B_BYTES;
      constexpr int NQ = Cfg::B_CHUNKS / N_LOW;
      float mx = 0.f;
      float4 v[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        v[q] = *reinterpret_cast<const float4*>(raw + (uint32_t)(t + q * N_LOW) * 16u);
        mx = fmaxf(fmaxf(mx, fmaxf(fabsf(v[q].x), fabsf(v[q].y))), fmaxf(fabsf(v[q].z), fabsf(v[q].w)));
      }
      const bool special = mx == INFINITY;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        float4 l;
        if (special) l = make_float4(lo1_safe(v[q].x), lo1_safe(v[q].y), lo1_safe(v[q].z), lo1_safe(v[q].w));
        else l = make_float4(lo1(v[q].x), lo1(v[q].y), lo1(v[q].z), lo1(v[q].w));
        *reinterpret_cast<float4*>(low + (uint32_t)(t + q * N_LOW) * 16u) = l;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(smem_u32(&b_ready[s]));
    }
  } else {
    // ------------------------------ MMA issuer (whole warp, one elected lane issues) --------------------------
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((B_KCONTIG ? 0u : 1u) << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TBM >> 4) << 24);
    const uint32_t base0 = smem_u32(smem) + Cfg::A_BYTES;
    const uint64_t d_b = B_KCONTIG ? umma_desc(base0) : umma_desc_mn(base0, BN / 32);
    constexpr uint64_t LOW = (uint64_t)(Cfg::B_BYTES >> 4);
    constexpr uint64_t B_STEP = (uint64_t)((B_KCONTIG ? 32 : (BN / 32) * 1024) >> 4);
    for (int j = 0; j < ktiles; ++j) {
      const int s = j % S;
      const uint32_t ph = (uint32_t)((j / S) & 1);
      const bool ok = !*failed && mbar_wait(smem_u32(&a_ready[s]), ph) && mbar_wait(smem_u32(&b_ready[s]), ph);
      if (!__all_sync(0xFFFFFFFFu, ok)) { *failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t st = (uint64_t)((s * Cfg::STAGE_BYTES) >> 4);
      const uint32_t a_hi = tmem + (uint32_t)(Cfg::A_COL0 + s * 64);
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < TBK / 8; ++kk) {
          const uint64_t db = d_b + st + kk * B_STEP;
          umma_tf32_ta(tmem, a_hi + kk * 8, db, idesc, (j | kk) != 0);
          umma_tf32_ta(tmem, a_hi + kk * 8, db + LOW, idesc, 1);
          umma_tf32_ta(tmem, a_hi + 32 + kk * 8, db, idesc, 1);
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty[s]))
                     : "memory");
      }
      __syncwarp();
    }
    // The read-back warps may reach their wait several k-tiles early, so they cannot use a stage barrier (a
    // parity wait is only unambiguous within one phase): a last commit completes `done` exactly once.
    if (elect_one())
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(done)) : "memory");
    __syncwarp();
  }

  if (warp >= W_CONV && warp < W_LOW) {
    // a warp can only read the tensor-memory lanes of quadrant warp % 4; the converter group picks the column half
    const int ew = (warp & 3) + 4 * ((warp - W_CONV) >> 2);
    store_accumulator<BN>(tmem, ew, lane, m0, n0, g, sp, ktiles, p, C, partial, c_row, c_col, c_grp, failed,
                          smem_u32(done), 0u);
    if (CONV_GROUPS == 1)                            // four read-back warps: each also takes the second column half
      store_accumulator<BN>(tmem, ew + 4, lane, m0, n0, g, sp, ktiles, p, C, partial, c_row, c_col, c_grp, failed,
                            smem_u32(done), 0u);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *failed) atomicAdd(error_flag, 1);
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Row scatter, deterministic: updates are ranked by (row index, update number) with an all-pairs count, then one
// block per run of equal row indices applies the run's updates in update order, accumulating in fp32 and rounding
// to the element type once (the same result whatever the launch order). Out-of-range indices are dropped.
template <typename I>
__global__ void __launch_bounds__(256) scatter_rank_kernel(const I* __restrict__ idx, int U, long long rows, int* __restrict__ key,
                                                         int* __restrict__ order) {
  const int u = blockIdx.x * 256 + threadIdx.x;
  if (u >= U) return;
  auto key_of = [&](int v) -> long long {
    const long long r = (long long)idx[v];
    return (r < 0 || r >= rows) ? rows : r;            // dropped updates sort to the end
  };
  const long long mine = key_of(u);
  int rank = 0;
  for (int v = 0; v < U; ++v) {
    const long long kv = key_of(v);
    rank += (kv < mine || (kv == mine && v < u)) ? 1 : 0;
  }
  order[rank] = u;
  key[rank] = (int)mine;
}

// The same ranking for many updates: a stable least-significant-digit radix sort of (row index, update number) with
// 8-bit digits, 1024 elements per block. Per pass: digit histograms per block, one exclusive scan over (digit, block),
// then every element goes to scan[digit][block] + the number of earlier elements of its block with the same digit
// (within a warp by matching lanes, across the block's warps by a table of per-warp counts): equal keys keep their
// update order, which is what makes the accumulation order, and so the result, independent of the launch.
template <typename I>
__global__ void __launch_bounds__(256) scatter_keys_kernel(const I* __restrict__ idx, int U, long long rows, int* __restrict__ key,
                                                         int* __restrict__ val) {
  const int u = blockIdx.x * 256 + threadIdx.x;
  if (u >= U) return;
  const long long r = (long long)idx[u];
  key[u] = (r < 0 || r >= rows) ? (int)rows : (int)r;          // dropped updates sort to the end
  val[u] = u;
}

__global__ void __launch_bounds__(1024) radix_hist_kernel(const int* __restrict__ key, int U, int shift, int* __restrict__ hist, int nblocks) {
  __shared__ int h[256];
  if (threadIdx.x < 256) h[threadIdx.x] = 0;
  __syncthreads();
  const int e = blockIdx.x * 1024 + threadIdx.x;
  if (e < U) atomicAdd(&h[((unsigned)key[e] >> shift) & 255u], 1);
  __syncthreads();
  if (threadIdx.x < 256) hist[threadIdx.x * nblocks + blockIdx.x] = h[threadIdx.x];
}

// exclusive scan of n integers in place by one block: a contiguous chunk per thread, the chunk sums scanned in shared memory
__global__ void __launch_bounds__(1024) radix_scan_kernel(int* __restrict__ hist, int n) {
  __shared__ int sums[1024];
  const int per = (n + 1023) / 1024;
  const int lo = min(n, (int)threadIdx.x * per), hi = min(n, lo + per);
  int s = 0;
  for (int i = lo; i < hi; ++i) s += hist[i];
  sums[threadIdx.x] = s;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int v = threadIdx.x >= off ? sums[threadIdx.x - off] : 0;
    __syncthreads();
    sums[threadIdx.x] += v;
    __syncthreads();
  }
  int run = sums[threadIdx.x] - s;
  for (int i = lo; i < hi; ++i) {
    const int v = hist[i];
    hist[i] = run;
    run += v;
  }
}

__global__ void __launch_bounds__(1024) radix_scatter_kernel(const int* __restrict__ key_in, const int* __restrict__ val_in,
                                                           int* __restrict__ key_out, int* __restrict__ val_out, int U, int shift,
                                                           const int* __restrict__ offsets, int nblocks) {
  __shared__ int cnt[32][256];
  for (int q = threadIdx.x; q < 32 * 256; q += 1024) (&cnt[0][0])[q] = 0;
  __syncthreads();
  const int e = blockIdx.x * 1024 + threadIdx.x, w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool valid = e < U;
  const int k = valid ? key_in[e] : 0, v = valid ? val_in[e] : 0;
  const int d = valid ? (int)(((unsigned)k >> shift) & 255u) : -1 - lane;     // lanes past the end match nobody
  const unsigned peers = __match_any_sync(0xFFFFFFFFu, d);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  if (valid && rank == 0) cnt[w][d] = __popc(peers);
  __syncthreads();
  if (threadIdx.x < 256) {
    int run = offsets[threadIdx.x * nblocks + blockIdx.x];
    for (int q = 0; q < 32; ++q) {
      const int c = cnt[q][threadIdx.x];
      cnt[q][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
  if (valid) {
    const int pos = cnt[w][d] + rank;
    key_out[pos] = k;
    val_out[pos] = v;
  }
}

__device__ __forceinline__ float scatter_load(const float* p) { return *p; }
__device__ __forceinline__ float scatter_load(const unsigned short* p) { return __uint_as_float((uint32_t)*p << 16); }
__device__ __forceinline__ int scatter_load(const int* p) { return *p; }
__device__ __forceinline__ void scatter_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void scatter_store(int* p, int v) { *p = v; }
__device__ __forceinline__ unsigned short bf16_round(float v) {
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (unsigned short)((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (unsigned short)(u >> 16);
}
__device__ __forceinline__ void scatter_store(unsigned short* p, float v) { *p = bf16_round(v); }

template <typename T, typename A>
__global__ void __launch_bounds__(256) scatter_apply_kernel(T* __restrict__ out, const T* __restrict__ upd, const int* __restrict__ key,
                                                          const int* __restrict__ order, int U, long long rows,
                                                          long long row_elems, int kind) {
  const int p = blockIdx.x;
  const int row = key[p];
  if (row >= rows || (p > 0 && key[p - 1] == row)) return;      // not the start of a run
  int end = p + 1;
  while (end < U && key[end] == row) ++end;
  for (long long d = (long long)blockIdx.y * 256 + threadIdx.x; d < row_elems; d += 256ll * gridDim.y) {
    A acc = scatter_load(out + (long long)row * row_elems + d);
    for (int q = p; q < end; ++q) {
      const A v = scatter_load(upd + (long long)order[q] * row_elems + d);
      A r;
      switch (kind) {
        case 0: r = v; break;
        case 1: r = acc + v; break;
        case 2: r = acc * v; break;
        case 3: r = (v < acc || v != v) ? v : acc; break;
        default: r = (v > acc || v != v) ? v : acc; break;
      }
      acc = r;
    }
    scatter_store(out + (long long)row * row_elems + d, acc);
  }
}

// General scatter: (destination element, update element) pairs sorted by destination, ties in update order; one
// thread per run of equal destinations folds the run's updates into the element in that order.
template <typename T, typename A>
__global__ void __launch_bounds__(256) scatter_apply_elems_kernel(T* __restrict__ out, const T* __restrict__ upd, const int* __restrict__ key,
                                                                const int* __restrict__ order, int U, long long numel, int kind) {
  const int p = blockIdx.x * 256 + threadIdx.x;
  if (p >= U) return;
  const int dest = key[p];
  if (dest >= numel || (p > 0 && key[p - 1] == dest)) return;
  A acc = scatter_load(out + dest);
  for (int q = p; q < U && key[q] == dest; ++q) {
    const A v = scatter_load(upd + order[q]);
    A r;
    switch (kind) {
      case 0: r = v; break;
      case 1: r = acc + v; break;
      case 2: r = acc * v; break;
      case 3: r = (v < acc || v != v) ? v : acc; break;
      default: r = (v > acc || v != v) ? v : acc; break;
    }
    acc = r;
  }
  scatter_store(out + dest, acc);
}

}  // namespace

cudaError_t launch_igemm_f32(const IGemmLaunch& p, const void* A, const void* B, void* C, const void* const* tables,
                             void* partial, const int* kt_table, int* error_flag, cudaStream_t stream, int* launches) {
  auto a_row = (const RowEnt*)tables[0];
  auto a_col = (const ColEnt*)tables[1];
  auto b_row = (const long long*)tables[2];
  auto b_col = (const long long*)tables[3];
  auto c_row = (const long long*)tables[4];
  auto c_col = (const long long*)tables[5];
  auto a_grp = (const long long*)tables[6];
  auto b_grp = (const long long*)tables[7];
  auto c_grp = (const long long*)tables[8];
  int v = (p.a_mcontig ? 4 : 0) | (p.b_kcontig ? 2 : 0) | (p.mask ? 1 : 0);
  if (p.tensor_cores) {
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
#define SETATTR(AM, BK_, MK) \
  cudaFuncSetAttribute(igemm_tf32x3_kernel<AM, BK_, MK>, cudaFuncAttributeMaxDynamicSharedMemorySize, TSMEM_BYTES)
      SETATTR(false, false, false); SETATTR(false, false, true); SETATTR(false, true, false); SETATTR(false, true, true);
      SETATTR(true, false, false); SETATTR(true, false, true); SETATTR(true, true, false); SETATTR(true, true, true);
#undef SETATTR
    }
    dim3 grid((p.M + TBM - 1) / TBM, (p.N + TBN - 1) / TBN, p.groups * p.split_k);
    if (p.vec) {
      static bool configured_w[64] = {};
      if (first_use_on_this_device(configured_w)) {
#define SETATTRW(BN_, AM, BK_, MK)                                                                                    \
  cudaFuncSetAttribute(igemm_tf32x3_ws_kernel<BN_, AM, BK_, MK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                       WsCfg<BN_>::SMEM);                                                                            \
  cudaFuncSetAttribute(igemm_tf32x3_ws_kernel<BN_, AM, BK_, MK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                       WsCfg<BN_>::SMEM);                                                                            \
  cudaFuncSetAttribute(igemm_tf32x3_ta_kernel<BN_, AM, BK_, MK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                       TaCfg<BN_, false>::SMEM);                                                                     \
  cudaFuncSetAttribute(igemm_tf32x3_ta_kernel<64, AM, BK_, MK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                       TaCfg<64, true>::SMEM)
#define SETALLW(BN_)                                                                                                  \
  SETATTRW(BN_, false, false, false); SETATTRW(BN_, false, false, true); SETATTRW(BN_, false, true, false);           \
  SETATTRW(BN_, false, true, true); SETATTRW(BN_, true, false, false); SETATTRW(BN_, true, false, true);              \
  SETATTRW(BN_, true, true, false); SETATTRW(BN_, true, true, true)
        SETALLW(64);
        SETALLW(128);
#undef SETALLW
#undef SETATTRW
      }
      alignas(64) CUtensorMap tm_a;
      memset(&tm_a, 0, sizeof tm_a);
      IGemmLaunch pl = p;
      if (p.a_tma && p.seg && p.tmem_a) {
        const unsigned long long dims[4] = {(unsigned long long)p.tma_c, (unsigned long long)p.tma_w, (unsigned long long)p.tma_h,
                                            (unsigned long long)p.tma_n};
        const unsigned long long strides[3] = {4ull * p.tma_c, 4ull * p.tma_c * p.tma_w, 4ull * p.tma_c * p.tma_w * p.tma_h};
        const unsigned box[4] = {(unsigned)TBK, (unsigned)p.tma_ow, (unsigned)p.tma_box_h, (unsigned)p.tma_box_n};
        if (!encode_tensor_map(&tm_a, 2, 4, A, dims, strides, box)) pl.a_tma = 0;      // fall back to the gather
      } else pl.a_tma = 0;
      const bool wide = p.N >= 128 && p.wide_n;
      // two half-size CTAs per SM for 64-wide tiles once the grid has more than one wave of full-size CTAs
      const long long ctas64 = (long long)((p.M + TBM - 1) / TBM) * ((p.N + 63) / 64) * p.groups * p.split_k;
      const bool half = !wide && p.half_ctas && ctas64 > 148;
      dim3 gridw((p.M + TBM - 1) / TBM, (p.N + (wide ? 128 : 64) - 1) / (wide ? 128 : 64), p.groups * p.split_k);
#define LAUNCHW(BN_, AM, BK_, MK)                                                                                     \
  if (p.seg && p.tmem_a && half)                                                                                      \
    launch_k(igemm_tf32x3_ta_kernel<64, AM, BK_, MK, true>, gridw, TaCfg<64, true>::THREADS, TaCfg<64, true>::SMEM, stream,  \
        (const float*)A, (const float*)B, (float*)C, a_row, a_col, b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp,     \
        (float*)partial, kt_table, error_flag, tm_a, pl);                                                             \
  else if (p.seg && p.tmem_a)                                                                                         \
    launch_k(igemm_tf32x3_ta_kernel<BN_, AM, BK_, MK, false>, gridw, TaCfg<BN_, false>::THREADS, TaCfg<BN_, false>::SMEM, stream,  \
        (const float*)A, (const float*)B, (float*)C, a_row, a_col, b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp,     \
        (float*)partial, kt_table, error_flag, tm_a, pl);                                                             \
  else if (p.seg)                                                                                                     \
    launch_k(igemm_tf32x3_ws_kernel<BN_, AM, BK_, MK, true>, gridw, WS_THREADS, WsCfg<BN_>::SMEM, stream,                   \
        (const float*)A, (const float*)B, (float*)C, a_row, a_col, b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp,     \
        (float*)partial, error_flag, p);                                                                              \
  else                                                                                                                \
    launch_k(igemm_tf32x3_ws_kernel<BN_, AM, BK_, MK, false>, gridw, WS_THREADS, WsCfg<BN_>::SMEM, stream,                  \
        (const float*)A, (const float*)B, (float*)C, a_row, a_col, b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp,     \
        (float*)partial, error_flag, p)
#define SWITCHW(BN_)                                   \
  switch (v) {                                         \
    case 0: LAUNCHW(BN_, false, false, false); break;  \
    case 1: LAUNCHW(BN_, false, false, true); break;   \
    case 2: LAUNCHW(BN_, false, true, false); break;   \
    case 3: LAUNCHW(BN_, false, true, true); break;    \
    case 4: LAUNCHW(BN_, true, false, false); break;   \
    case 5: LAUNCHW(BN_, true, false, true); break;    \
    case 6: LAUNCHW(BN_, true, true, false); break;    \
    default: LAUNCHW(BN_, true, true, true); break;    \
  }
      if (wide) { SWITCHW(128) } else { SWITCHW(64) }
#undef SWITCHW
#undef LAUNCHW
    } else {
#define LAUNCHT(AM, BK_, MK)                                                                                     \
  launch_k(igemm_tf32x3_kernel<AM, BK_, MK>, grid, TNT, TSMEM_BYTES, stream, (const float*)A, (const float*)B, (float*)C, \
                                                                        a_row, a_col, b_row, b_col, c_row, c_col,   \
                                                                        a_grp, b_grp, c_grp, (float*)partial,       \
                                                                        error_flag, p)
    switch (v) {
      case 0: LAUNCHT(false, false, false); break;
      case 1: LAUNCHT(false, false, true); break;
      case 2: LAUNCHT(false, true, false); break;
      case 3: LAUNCHT(false, true, true); break;
      case 4: LAUNCHT(true, false, false); break;
      case 5: LAUNCHT(true, false, true); break;
      case 6: LAUNCHT(true, true, false); break;
      default: LAUNCHT(true, true, true); break;
    }
#undef LAUNCHT
    }
  } else {
    dim3 grid((p.M + BM - 1) / BM, (p.N + BN - 1) / BN, p.groups * p.split_k);
    dim3 block(NT);
#define LAUNCH(AM, BK_, MK)                                                                                          \
  launch_k(igemm_f32_kernel<AM, BK_, MK>, grid, block, 0, stream, (const float*)A, (const float*)B, (float*)C, a_row, a_col, \
                                                            b_row, b_col, c_row, c_col, a_grp, b_grp, c_grp,           \
                                                            (float*)partial, p)
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
  }
  if (launches) (*launches)++;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (p.split_k > 1) {
    long long total = (long long)p.groups * p.M * p.N;
    // four consecutive n per thread when they are four consecutive, 16-byte aligned floats of C; the splits are
    // spread over 8 thread rows when there are many of them and few outputs
    const float* pp = (const float*)partial;
    float* cc = (float*)C;
    const bool vec = p.c_vec == 2 && p.N % 4 == 0 && (((uintptr_t)C) & 15) == 0 && (((uintptr_t)partial) & 15) == 0;
    const long long items = vec ? total / 4 : total;
    const bool tall = p.split_k >= 16;
    const unsigned blocks = (unsigned)(tall ? (items + 31) / 32 : (items + 255) / 256);
    if (vec && tall) launch_k(splitk_reduce_kernel<8, true>, blocks, dim3(32, 8), 0, stream, pp, cc, c_row, c_col, c_grp, p.M, p.N, p.groups, p.split_k);
    else if (vec) launch_k(splitk_reduce_kernel<1, true>, blocks, dim3(256, 1), 0, stream, pp, cc, c_row, c_col, c_grp, p.M, p.N, p.groups, p.split_k);
    else if (tall) launch_k(splitk_reduce_kernel<8, false>, blocks, dim3(32, 8), 0, stream, pp, cc, c_row, c_col, c_grp, p.M, p.N, p.groups, p.split_k);
    else launch_k(splitk_reduce_kernel<1, false>, blocks, dim3(256, 1), 0, stream, pp, cc, c_row, c_col, c_grp, p.M, p.N, p.groups, p.split_k);
    if (launches) (*launches)++;
    e = cudaGetLastError();
  }
  return e;
}


// ---------------------------------------------------------------------------
// Split-K fp32 matrix product whose scratch lives in the library image instead of an allocation.
//
// Some callers may not allocate device memory at the moment they need a product: code running inside a
// memory-pool callback or under a framework allocator lock, a library initialiser that must not disturb the
// process's memory accounting, a real-time loop that forbids anything that can take the driver's allocation
// lock. For them the partial sums of the K splits go to a file-scope device array (8 MiB, resident on every
// GPU that loads this library until the process exits) rather than to arena or pool memory.
namespace {

constexpr size_t kStaticScratchFloats = 2u << 20;                    // 8 MiB
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int SBM = 64, SBN = 64, SBK = 16;

// C partial [split][M][N] = A[M, k-range] * B[k-range, N]; dense row-major operands, 256 threads, 4 x 4 per thread.
__global__ void __launch_bounds__(256) matmul_splitk_static_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                                  float* __restrict__ partial, int M, int N, int K,
                                                                  int splits) {
  __shared__ float As[SBK][SBM + 1];
  __shared__ float Bs[SBK][SBN + 1];
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * SBM, n0 = blockIdx.y * SBN, sp = blockIdx.z;
  const int kchunk = ((K + splits - 1) / splits + SBK - 1) / SBK * SBK;
  const int kbeg = sp * kchunk, kend = min(K, kbeg + kchunk);
  float acc[4][4] = {};
  for (int k0 = kbeg; k0 < kend; k0 += SBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int idx = tid + 256 * i;                      // 1024 elements of each tile
      int am = idx / SBK, ak = idx % SBK;
      As[ak][am] = (m0 + am < M && k0 + ak < kend) ? A[(size_t)(m0 + am) * K + k0 + ak] : 0.f;
      int bk = idx / SBN, bn = idx % SBN;
      Bs[bk][bn] = (k0 + bk < kend && n0 + bn < N) ? B[(size_t)(k0 + bk) * N + n0 + bn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < SBK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* out = partial + (size_t)sp * M * N;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) out[(size_t)m * N + n] = acc[i][j];      // every element of the split's slab is written
    }
}

__global__ void __launch_bounds__(256) splitk_sum_static_kernel(const float* __restrict__ partial, float* __restrict__ C,
                                                               long long total, int splits) {
  long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += partial[(long long)k * total + i];
  C[i] = s;
}

}  // namespace

size_t static_scratch_bytes() { return kStaticScratchFloats * sizeof(float); }

cudaError_t matmul_f32_static_scratch(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream,
                                      const char** why) {
  *why = nullptr;
  // The array's name is a host-side handle; kernels need its device address, which differs per device.
  static float* scratch_of_device[64] = {};
  static bool resolved[64] = {};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) { *why = "device ordinal out of range"; return cudaErrorInvalidDevice; }
  std::lock_guard<std::mutex> lock(mu);     // guards the address cache and serialises the enqueueing; launches that overlap on the GPU still race
  if (!resolved[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) { *why = "cudaGetSymbolAddress(g_static_scratch) failed"; return e; }
    scratch_of_device[dev] = (float*)ptr;
    resolved[dev] = true;
  }
  float* scratch = scratch_of_device[dev];
  const long long mn = (long long)M * N;
  int splits = (int)std::min<long long>(std::max(2, (K + 255) / 256), 32);
  while (splits > 2 && (long long)splits * mn > (long long)kStaticScratchFloats) splits--;
  if ((long long)splits * mn > (long long)kStaticScratchFloats) {
    *why = "M * N is too large for the static scratch (two K splits of M * N floats must fit in 8 MiB)";
    return cudaErrorInvalidValue;
  }
  dim3 grid((M + SBM - 1) / SBM, (N + SBN - 1) / SBN, splits);
  matmul_splitk_static_kernel<<<grid, 256, 0, stream>>>(A, B, scratch, M, N, K, splits);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  splitk_sum_static_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, stream>>>(scratch, C, mn, splits);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Probe: the rate at which the tensor cores retire tcgen05.mma.kind::tf32 on this GPU, measured with the issue loop
// alone (operands resident in shared memory, nothing to load): the ceiling of the three-MMA fp32-accurate scheme is a
// third of it. One CTA per SM, 128 x 128 x 8 MMAs, `iters` groups of 12 per CTA.
namespace {
__global__ void __launch_bounds__(128, 1) tf32_mma_rate_kernel(int iters, int* __restrict__ error_flag) {
  extern __shared__ uint8_t probe_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)probe_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bars[2];
  __shared__ uint32_t tmem_slot;
  constexpr int A_BYTES = 128 * 32 * 4, B_BYTES = 128 * 32 * 4;
  const int tid = threadIdx.x;
  float* f = (float*)smem;
  for (int i = tid; i < (A_BYTES + B_BYTES) / 4; i += 128) f[i] = 1.0f + (i % 7) * 0.125f;
  if (tid == 0) {
    mbar_init(smem_u32(&bars[0]), 1);
    mbar_init(smem_u32(&bars[1]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 32) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(128) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    const uint64_t d_a = umma_desc(smem_u32(smem)), d_b = umma_desc(smem_u32(smem) + A_BYTES);
    for (int j = 0; j < iters; ++j) {
#pragma unroll
      for (int q = 0; q < 12; ++q) umma_tf32(tmem, d_a + (uint64_t)((q & 3) * 2), d_b + (uint64_t)((q & 3) * 2), idesc, (j | q) != 0);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bars[j == iters - 1]))
                   : "memory");
    }
    if (!mbar_wait(smem_u32(&bars[1]), 0)) atomicAdd(error_flag, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128) : "memory");
}
}  // namespace

namespace {
// Test hook: a wait on an mbarrier that nothing ever arrives at, with a small poll budget. It runs out, and the
// kernel reports it exactly as the tensor-core kernels report an expired pipeline wait: it counts up the error word
// and returns. Nothing hangs and nothing faults.
__global__ void expiring_wait_kernel(int polls, int* __restrict__ error_flag) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    bool done = false;
    for (int spin = 0; spin < polls && !done; ++spin) {
      uint32_t ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(smem_u32(&bar)), "r"(0u)
          : "memory");
      done = ok != 0;
    }
    if (!done) atomicAdd(error_flag, 1);
  }
}
}  // namespace

// ---------------------------------------------------------------------------
// Conditional graph nodes: the kernels that set a node's handle from a value on the device, so that a data-dependent
// `while` or `case` needs no host round trip. The while form is bounded in time: `*started` holds the loop's start
// (written when `first`), and once `limit_ns` has passed the loop ends and the error counter goes up.
namespace {
__global__ void while_handle_kernel(cudaGraphConditionalHandle handle, const unsigned char* __restrict__ pred,
                                    unsigned long long* __restrict__ started, unsigned long long limit_ns, int first,
                                    int* __restrict__ error_flag) {
  unsigned long long now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
  if (first) *started = now;
  unsigned int go = *pred != 0 ? 1u : 0u;
  if (go && now - *started > limit_ns) {
    go = 0u;
    atomicAdd(error_flag, 1);
  }
  cudaGraphSetConditional(handle, go);
}
__global__ void switch_handle_kernel(cudaGraphConditionalHandle handle, const int* __restrict__ index, int branches) {
  const int i = *index;
  cudaGraphSetConditional(handle, (unsigned int)((i < 0 || i >= branches) ? branches - 1 : i));   // out of range: the last branch
}
}  // namespace

cudaError_t launch_while_handle(unsigned long long handle, const void* pred, unsigned long long* started, double limit_seconds,
                                bool first, int* error_flag, cudaStream_t stream) {
  while_handle_kernel<<<1, 1, 0, stream>>>((cudaGraphConditionalHandle)handle, (const unsigned char*)pred, started,
                                           (unsigned long long)(limit_seconds * 1e9), first ? 1 : 0, error_flag);
  return cudaGetLastError();
}

cudaError_t launch_switch_handle(unsigned long long handle, const void* index, int branches, cudaStream_t stream) {
  switch_handle_kernel<<<1, 1, 0, stream>>>((cudaGraphConditionalHandle)handle, (const int*)index, branches);
  return cudaGetLastError();
}

cudaError_t launch_expiring_wait(int polls, int* error_flag, cudaStream_t stream) {
  expiring_wait_kernel<<<1, 32, 0, stream>>>(polls < 1 ? 1 : polls, error_flag);
  return cudaGetLastError();
}

cudaError_t probe_tf32_mma_rate(int* error_flag, cudaStream_t stream, double* tflops) {
  *tflops = 0.0;
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  constexpr int SMEM = 2 * 128 * 32 * 4 + 1024;
  e = cudaFuncSetAttribute(tf32_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) return e;
  cudaEvent_t a, b;
  cudaEventCreate(&a);
  cudaEventCreate(&b);
  const int iters = 4000;
  tf32_mma_rate_kernel<<<sms, 128, SMEM, stream>>>(100, error_flag);
  cudaEventRecord(a, stream);
  tf32_mma_rate_kernel<<<sms, 128, SMEM, stream>>>(iters, error_flag);
  cudaEventRecord(b, stream);
  e = cudaStreamSynchronize(stream);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, a, b);
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  if (e != cudaSuccess) return e;
  *tflops = 2.0 * 128 * 128 * 8 * 12.0 * iters * sms / (ms * 1e-3) / 1e12;
  return cudaGetLastError();
}

constexpr int kScatterAllPairsMax = 1024;          // up to here the all-pairs ranking (one launch) is the quicker one
static int scatter_radix_passes(long long rows);

cudaError_t launch_scatter_rows(int elem_kind, int index_bytes, int kind, long long rows, long long row_elems, int updates,
                                void* out, const void* indices, const void* upd, int* scratch, cudaStream_t stream,
                                int* launches) {
  if (updates <= 0 || rows <= 0 || row_elems <= 0) return cudaSuccess;
  int* key = scratch;
  int* order = scratch + updates;
  const unsigned rb = (unsigned)((updates + 255) / 256);
  if (updates <= kScatterAllPairsMax) {
    if (index_bytes == 8)
      scatter_rank_kernel<long long><<<rb, 256, 0, stream>>>((const long long*)indices, updates, rows, key, order);
    else
      scatter_rank_kernel<int><<<rb, 256, 0, stream>>>((const int*)indices, updates, rows, key, order);
    *launches += 1;
  } else {
    int* key_b = scratch + 2 * (long long)updates;
    int* order_b = scratch + 3 * (long long)updates;
    int* hist = scratch + 4 * (long long)updates;
    const int nblocks = (updates + 1023) / 1024;
    if (index_bytes == 8)
      scatter_keys_kernel<long long><<<rb, 256, 0, stream>>>((const long long*)indices, updates, rows, key, order);
    else
      scatter_keys_kernel<int><<<rb, 256, 0, stream>>>((const int*)indices, updates, rows, key, order);
    const int passes = scatter_radix_passes(rows);
    for (int pass = 0; pass < passes; ++pass) {
      radix_hist_kernel<<<nblocks, 1024, 0, stream>>>(key, updates, 8 * pass, hist, nblocks);
      radix_scan_kernel<<<1, 1024, 0, stream>>>(hist, 256 * nblocks);
      radix_scatter_kernel<<<nblocks, 1024, 0, stream>>>(key, order, key_b, order_b, updates, 8 * pass, hist, nblocks);
      std::swap(key, key_b);
      std::swap(order, order_b);
    }
    *launches += 1 + 3 * passes;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dim3 grid((unsigned)updates, (unsigned)std::min<long long>(64, (row_elems + 255) / 256));
  if (elem_kind == 0)
    scatter_apply_kernel<float, float><<<grid, 256, 0, stream>>>((float*)out, (const float*)upd, key, order, updates, rows, row_elems, kind);
  else if (elem_kind == 1)
    scatter_apply_kernel<unsigned short, float><<<grid, 256, 0, stream>>>((unsigned short*)out, (const unsigned short*)upd, key, order,
                                                                          updates, rows, row_elems, kind);
  else
    scatter_apply_kernel<int, int><<<grid, 256, 0, stream>>>((int*)out, (const int*)upd, key, order, updates, rows, row_elems, kind);
  *launches += 1;
  return cudaGetLastError();
}

cudaError_t launch_scatter_elems(int elem_kind, int kind, long long numel, int updates, void* out, const void* upd, int* scratch,
                                 cudaStream_t stream, int* launches) {
  if (updates <= 0 || numel <= 0) return cudaSuccess;
  int *key = scratch, *order = scratch + updates;
  int *key_b = scratch + 2 * (long long)updates, *order_b = scratch + 3 * (long long)updates, *hist = scratch + 4 * (long long)updates;
  const int nblocks = (updates + 1023) / 1024;
  const int passes = scatter_radix_passes(numel);
  for (int pass = 0; pass < passes; ++pass) {
    radix_hist_kernel<<<nblocks, 1024, 0, stream>>>(key, updates, 8 * pass, hist, nblocks);
    radix_scan_kernel<<<1, 1024, 0, stream>>>(hist, 256 * nblocks);
    radix_scatter_kernel<<<nblocks, 1024, 0, stream>>>(key, order, key_b, order_b, updates, 8 * pass, hist, nblocks);
    std::swap(key, key_b);
    std::swap(order, order_b);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (kind < 0) {                        // sort only: a generated kernel applies the update computation
    *launches += 3 * passes;
    return cudaSuccess;
  }
  const unsigned grid = (unsigned)((updates + 255) / 256);
  if (elem_kind == 0)
    scatter_apply_elems_kernel<float, float><<<grid, 256, 0, stream>>>((float*)out, (const float*)upd, key, order, updates, numel, kind);
  else if (elem_kind == 1)
    scatter_apply_elems_kernel<unsigned short, float><<<grid, 256, 0, stream>>>((unsigned short*)out, (const unsigned short*)upd, key, order,
                                                                                updates, numel, kind);
  else
    scatter_apply_elems_kernel<int, int><<<grid, 256, 0, stream>>>((int*)out, (const int*)upd, key, order, updates, numel, kind);
  *launches += 3 * passes + 1;
  return cudaGetLastError();
}

long long scatter_elems_scratch_ints(long long updates) {
  updates = std::max<long long>(updates, 1);
  return 4 * updates + 256 * ((updates + 1023) / 1024);
}

int scatter_elems_launches(long long numel) { return 3 * scatter_radix_passes(numel) + 1; }

static int scatter_radix_passes(long long rows) {
  int bits = 1;
  while (bits < 32 && (1ll << bits) <= rows) ++bits;          // keys lie in [0, rows]
  return (bits + 7) / 8;
}

long long scatter_rows_scratch_ints(long long rows, long long updates) {
  updates = std::max<long long>(updates, 1);
  if (updates <= kScatterAllPairsMax) return 2 * updates;
  return 4 * updates + 256 * ((updates + 1023) / 1024);
}

int scatter_rows_launches(long long rows, long long updates) {
  return updates <= kScatterAllPairsMax ? 2 : 2 + 3 * scatter_radix_passes(rows);
}

void set_igemm_programmatic_launch(bool on) { g_igemm_programmatic_launch = on; }

}  // namespace b200
