// Contractions of 16-bit floating-point operands (bf16 / f16): what stablehlo.dot_general lowers to when both
// operands are half precision (the reference forwards these to MLX: src/pjrt_plugin/ops/linalg.cc:89-250).
// Products are exact in fp32, accumulation is fp32, the result is rounded once to its element type.
//
//   gemm16_tma_kernel   tensor-core tiles for M > 8. One persistent CTA per SM walks the output tiles. Warp 0 moves
//                       operand tiles with TMA tiled copies (cp.async.bulk.tensor, this GPU's memory only, plain
//                       single-CTA form) into a ring of 128-byte-swizzled shared-memory stages; warp 1 issues
//                       tcgen05.mma.kind::f16 from shared-memory descriptors into one of two accumulators in tensor
//                       memory; warps 2-9 read a finished accumulator back (tcgen05.ld), round and store it while
//                       the next tile's products already run into the other accumulator.
//   gemv16_nc_kernel /  M <= 8 (a decode step): the weights are read exactly once with 128-bit loads and the rate is
//   gemv16_kc_kernel    set by HBM, so no tensor cores. nc: n contiguous in B; kc: k contiguous in B.
//
// Every mbarrier wait is bounded; on expiry the CTA raises *error_flag, skips its stores, waits (bounded) for its
// copies in flight, releases its tensor memory and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <mutex>

#include "kernels.h"
#include "tc_util.cuh"

namespace b200 {

namespace {
// Launches with programmatic stream serialization (every kernel of this file starts with pdl_prologue): the launch
// latency and the scheduling of this kernel's first blocks overlap the end of the kernel in front of it.
// Measured: 7.15 -> 6.42 ms on the DistilBERT-shaped step, 5.18 -> 4.95 ms on the ResNet18 step; neutral inside the
// replayed graphs of loop bodies.
bool g_programmatic_launch = true;

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
  cfg.numAttrs = g_programmatic_launch ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<A>(args)...);
}


constexpr int G_BM = 128, G_BK = 64, G_THREADS = 320;   // TMA warp, MMA warp, eight read-back warps

template <int BN>
struct G16Cfg {
  static constexpr int A_BYTES = G_BM * G_BK * 2, B_BYTES = BN * G_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);       // 192 KB of operand stages
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 2 * BN;                                 // two accumulators
};

struct Gemm16Params {
  int M, N, K, G;
  int a_mn, b_mn;                 // operand stored with m (n) contiguous instead of k
  int split_k, kt_per_split;
  int in_fmt, c_kind;
  int mtiles, ntiles;
};

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One TMA tiled copy of a box of a rank-3 tensor (x innermost) into shared memory; completion is counted in bytes
// on `bar`. x times the element size must be a multiple of 16 bytes; parts of the box outside the tensor read zero.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Shared-memory matrix descriptor of an operand stored with m (n) contiguous, 16-bit elements, 128-byte swizzle:
// atoms of 64 m x 8 k (8 rows of 128 bytes); 8-row groups along k are 1024 bytes apart (SBO), atoms along m are
// `atom_stride` bytes apart (LBO).
__device__ __forceinline__ uint64_t umma_desc_mn16(uint32_t smem_addr, uint32_t atom_stride) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)(atom_stride >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&v)[32]) {
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
}

// fp32 -> 16-bit, round to nearest even (NaN stays NaN)
__device__ __forceinline__ uint32_t to_bf16_bits(float v) {
  uint32_t u = __float_as_uint(v);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (u >> 16) | 0x40u;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return u >> 16;
}
__device__ __forceinline__ uint32_t to_f16_bits(float v) { return (uint32_t)__half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ uint32_t to16(float v, int c_kind) { return c_kind == 1 ? to_bf16_bits(v) : to_f16_bits(v); }

// Stores 32 consecutive columns (n0 ..) of row `row` of a dense [rows][N] result: fp32 as it is, 16-bit rounded. The
// widest store the row's address allows is used (a row of an odd-sized result starts 4 or 8 bytes off a 16-byte line).
__device__ __forceinline__ void store_row32(void* C, long long row, int N, int n0, const uint32_t (&v)[32], int c_kind) {
  if (n0 >= N) return;
  const bool full = n0 + 32 <= N;
  if (c_kind == 2) {
    float* out = (float*)C + row * N + n0;
    if (full && (((uintptr_t)out) & 15) == 0) {
#pragma unroll
      for (int q = 0; q < 32; q += 4)
        *reinterpret_cast<uint4*>(out + q) = make_uint4(v[q], v[q + 1], v[q + 2], v[q + 3]);
    } else {
#pragma unroll
      for (int q = 0; q < 32; ++q)
        if (n0 + q < N) out[q] = __uint_as_float(v[q]);
    }
    return;
  }
  uint16_t* out = (uint16_t*)C + row * N + n0;
  uint32_t w[16];
#pragma unroll
  for (int q = 0; q < 16; ++q) w[q] = to16(__uint_as_float(v[2 * q]), c_kind) | (to16(__uint_as_float(v[2 * q + 1]), c_kind) << 16);
  const uintptr_t a = (uintptr_t)out;
  if (full && (a & 15) == 0) {
#pragma unroll
    for (int q = 0; q < 16; q += 4) *reinterpret_cast<uint4*>(out + 2 * q) = make_uint4(w[q], w[q + 1], w[q + 2], w[q + 3]);
  } else if (full && (a & 7) == 0) {
#pragma unroll
    for (int q = 0; q < 16; q += 2) *reinterpret_cast<uint2*>(out + 2 * q) = make_uint2(w[q], w[q + 1]);
  } else if (full && (a & 3) == 0) {
#pragma unroll
    for (int q = 0; q < 16; ++q) *reinterpret_cast<uint32_t*>(out + 2 * q) = w[q];
  } else {
#pragma unroll
    for (int q = 0; q < 32; ++q)
      if (n0 + q < N) out[q] = (uint16_t)((q & 1) ? (w[q >> 1] >> 16) : (w[q >> 1] & 0xFFFFu));
  }
}

template <int BN>
__global__ void __launch_bounds__(G_THREADS, 1) gemm16_tma_kernel(const __grid_constant__ CUtensorMap tm_a,
                                                                  const __grid_constant__ CUtensorMap tm_b,
                                                                  void* __restrict__ C, float* __restrict__ partial,
                                                                  int* __restrict__ error_flag, Gemm16Params p) {
  pdl_prologue();
  using Cfg = G16Cfg<BN>;
  constexpr int S = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + S * Cfg::STAGE_BYTES);     // a stage's copies have landed
  uint64_t* empty = full + S;                                    // the MMAs that read a stage have retired
  uint64_t* acc_full = empty + S;                                // all MMAs of a tile have retired
  uint64_t* acc_empty = acc_full + 2;                            // the read-back warps are done with an accumulator
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile int* failed = (volatile int*)(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(smem_u32(&full[s]), 1);
      mbar_init(smem_u32(&empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&acc_full[b]), 1);
      mbar_init(smem_u32(&acc_empty[b]), 8);
    }
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  const int ktiles = (p.K + G_BK - 1) / G_BK;
  const long long tiles = (long long)p.mtiles * p.ntiles * p.G * p.split_k;
  // tile t -> (m tile fastest, so that CTAs running side by side share one panel of B, then n tile, group, split)
  auto decode = [&](long long t, int& mt, int& nt, int& g, int& sp) {
    mt = (int)(t % p.mtiles); t /= p.mtiles;
    nt = (int)(t % p.ntiles); t /= p.ntiles;
    g = (int)(t % p.G);
    sp = (int)(t / p.G);
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (whole warp loops, one elected lane issues) -----------------
    uint32_t it = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
      int mt, nt, g, sp;
      decode(t, mt, nt, g, sp);
      const int m0 = mt * G_BM, n0 = nt * BN;
      const int kt_end = min(ktiles, (sp + 1) * p.kt_per_split);
      for (int kt = sp * p.kt_per_split; kt < kt_end; ++kt, ++it) {
        const int s = it % S;
        ok = !*failed && mbar_wait(smem_u32(&empty[s]), ((it / S) & 1) ^ 1);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) { *failed = 1; break; }
        if (elect_one()) {
          const uint32_t bar = smem_u32(&full[s]);
          mbar_expect_tx(bar, Cfg::STAGE_BYTES);
          const uint32_t a_dst = smem_u32(smem + s * Cfg::STAGE_BYTES), b_dst = a_dst + Cfg::A_BYTES;
          const int k0 = kt * G_BK;
          if (!p.a_mn) tma_load_3d(a_dst, &tm_a, bar, k0, m0, g);                 // box 64 k x 128 m
          else {
            tma_load_3d(a_dst, &tm_a, bar, m0, k0, g);                            // boxes 64 m x 64 k
            tma_load_3d(a_dst + 8192, &tm_a, bar, m0 + 64, k0, g);
          }
          if (!p.b_mn) tma_load_3d(b_dst, &tm_b, bar, k0, n0, g);                 // box 64 k x BN n
          else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_3d(b_dst + j * 8192, &tm_b, bar, n0 + 64 * j, k0, g);
          }
        }
        __syncwarp();
      }
    }
    if (*failed) {
      // copies issued into stages nobody consumed any more: wait for them before the shared memory goes away
      const uint32_t pending = it < (uint32_t)S ? it : (uint32_t)S;
      for (uint32_t j = it - pending; j < it; ++j) mbar_wait(smem_u32(&full[j % S]), (j / S) & 1);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ---------------------------------------------------------------
    // instruction descriptor: D fp32, A / B f16 (0) or bf16 (1), major-ness per operand, N, M = 128
    const uint32_t idesc = (1u << 4) | ((uint32_t)p.in_fmt << 7) | ((uint32_t)p.in_fmt << 10) | ((p.a_mn ? 1u : 0u) << 15) |
                           ((p.b_mn ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(G_BM >> 4) << 24);
    const uint32_t base0 = smem_u32(smem);
    const uint64_t d_a = p.a_mn ? umma_desc_mn16(base0, 8192) : umma_desc(base0);
    const uint64_t d_b = p.b_mn ? umma_desc_mn16(base0 + Cfg::A_BYTES, 8192) : umma_desc(base0 + Cfg::A_BYTES);
    // one k-step of 16: 32 bytes along the swizzled row (k contiguous) or two 8-row groups (m / n contiguous)
    const uint64_t a_step = (uint64_t)((p.a_mn ? 2048 : 32) >> 4), b_step = (uint64_t)((p.b_mn ? 2048 : 32) >> 4);
    uint32_t it = 0, tl = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tl) {
      int mt, nt, g, sp;
      decode(t, mt, nt, g, sp);
      const uint32_t ab = tl & 1;
      ok = !*failed && mbar_wait(smem_u32(&acc_empty[ab]), ((tl >> 1) & 1) ^ 1);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) { *failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_tmem = tmem + ab * BN;
      const int kt_beg = sp * p.kt_per_split, kt_end = min(ktiles, kt_beg + p.kt_per_split);
      for (int kt = kt_beg; kt < kt_end; ++kt, ++it) {
        const int s = it % S;
        ok = !*failed && mbar_wait(smem_u32(&full[s]), (it / S) & 1);
        ok = __all_sync(0xFFFFFFFFu, ok);
        if (!ok) { *failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t st = (uint64_t)((s * Cfg::STAGE_BYTES) >> 4);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < G_BK / 16; ++kk)
            umma_f16(d_tmem, d_a + st + kk * a_step, d_b + st + kk * b_step, idesc, (kt > kt_beg || kk > 0) ? 1u : 0u);
          umma_commit(smem_u32(&empty[s]));
        }
        __syncwarp();
      }
      if (ok && elect_one()) umma_commit(smem_u32(&acc_full[ab]));
      __syncwarp();
    }
  } else {
    // ------------------------------ accumulator read-back (warps 2-9: lane quadrant warp % 4, two warps per quadrant,
    // each with one half of the tile's columns: with four warps the read-back of a 128 x 256 tile took longer than the
    // 12 k-tiles of a K = 768 product and set that product's time) ------------------------------------------------
    const int quad = warp & 3, half = (warp - 2) >> 2;
    uint32_t tl = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++tl) {
      int mt, nt, g, sp;
      decode(t, mt, nt, g, sp);
      const uint32_t ab = tl & 1;
      ok = !*failed && mbar_wait(smem_u32(&acc_full[ab]), (tl >> 1) & 1);
      ok = __all_sync(0xFFFFFFFFu, ok);
      if (!ok) { *failed = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m = mt * G_BM + 32 * quad + lane;
      const int n0 = nt * BN;
      const bool split = p.split_k > 1;
      void* out = split ? (void*)partial : C;
      const long long row = split ? ((long long)sp * p.G + g) * p.M + m : (long long)g * p.M + m;
      const int kind = split ? 2 : p.c_kind;
#pragma unroll 1
      // rows of C that start off 16-byte lines (N not a multiple of 8) go out in narrow stores: there the second warp
      // of a quadrant only adds pressure, the first one takes every column
      const bool shared_cols = split || (p.N & 7) == 0;
      const int c_begin = shared_cols ? half * (BN / 2) : 0, c_end = shared_cols ? (half + 1) * (BN / 2) : (half == 0 ? BN : 0);
      if (c_begin >= c_end) {
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&acc_empty[ab]));
      }
      for (int c0 = c_begin; c0 < c_end; c0 += 32) {
        uint32_t v[32];
        tmem_load32(tmem + ((uint32_t)(32 * quad) << 16) + ab * BN + (uint32_t)c0, v);
        if (c0 + 32 == c_end) {
          // the accumulator is in registers: hand it back to the MMA warp before storing
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&acc_empty[ab]));
        }
        if (m < p.M) store_row32(out, row, p.N, n0 + c0, v, kind);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && *failed) atomicAdd(error_flag, 1);
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(Cfg::TMEM_COLS) : "memory");
  }
}

// Sum of the K splits in a fixed order, rounded once: partial [split][rows][N] fp32 -> C [rows][N].
__global__ void __launch_bounds__(256) splitk_sum16_kernel(const float* __restrict__ partial, void* __restrict__ C, long long total,
                                                          int splits, int c_kind) {
  pdl_prologue();
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += __ldcs(partial + (long long)k * total + i);
  if (c_kind == 2) ((float*)C)[i] = s;
  else ((uint16_t*)C)[i] = (uint16_t)to16(s, c_kind);
}

__global__ void __launch_bounds__(256) repack_rows16_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, long long rows,
                                                           long long cols, long long dst_ld, long long src_ld) {
  pdl_prologue();
  const long long r = blockIdx.y;
  for (long long c = (long long)blockIdx.x * 256 + threadIdx.x; c < cols; c += 256ll * gridDim.x)
    dst[r * dst_ld + c] = src[r * src_ld + c];
}

// Batched two-dimensional transpose dst[b][c][r] = src[b][r][c] staged through shared memory, so that both the reads
// (along c) and the writes (along r) are whole 128-byte lines. 4-byte elements: 32 x 32 tiles; 2-byte elements:
// 64 x 64 tiles moved as pairs (R and C even). Block (32, 8), grid (tiles along c, tiles along r, b).
__global__ void __launch_bounds__(256) transpose32_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, int R, int C,
                                                         long long dst_ld, long long src_bs, long long dst_bs) {
  pdl_prologue();
  __shared__ uint32_t tile[32][33];
  const long long sb = (long long)blockIdx.z * src_bs, db = (long long)blockIdx.z * dst_bs;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
#pragma unroll
  for (int j = threadIdx.y; j < 32; j += 8)
    if (r0 + j < R && c0 + threadIdx.x < C) tile[j][threadIdx.x] = src[sb + (long long)(r0 + j) * C + c0 + threadIdx.x];
  __syncthreads();
#pragma unroll
  for (int j = threadIdx.y; j < 32; j += 8)
    if (c0 + j < C && r0 + threadIdx.x < R) dst[db + (long long)(c0 + j) * dst_ld + r0 + threadIdx.x] = tile[threadIdx.x][j];
}

// 4-byte elements, 64 x 64 tiles moved as pairs: 256 contiguous bytes per row on both sides (DRAM likes the longer
// runs: 0.80 of the copy bandwidth against 0.44 with 32 x 32 tiles), R, C and the leading dimensions even.
__global__ void __launch_bounds__(256) transpose32x2_kernel(uint32_t* __restrict__ dst, const uint32_t* __restrict__ src, int R, int C,
                                                           long long dst_ld, long long src_bs, long long dst_bs) {
  pdl_prologue();
  __shared__ uint32_t tile[64][65];
  const long long sb = (long long)blockIdx.z * src_bs, db = (long long)blockIdx.z * dst_bs;
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
  uint2 v[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int r = r0 + threadIdx.y + 8 * q, c = c0 + 2 * threadIdx.x;
    v[q] = make_uint2(0, 0);
    if (r < R && c < C) v[q] = *reinterpret_cast<const uint2*>(src + sb + (long long)r * C + c);
  }
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    tile[threadIdx.y + 8 * q][2 * threadIdx.x] = v[q].x;
    tile[threadIdx.y + 8 * q][2 * threadIdx.x + 1] = v[q].y;
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const int j = threadIdx.y + 8 * q, c = c0 + j, r = r0 + 2 * threadIdx.x;
    if (c < C && r < R)
      *reinterpret_cast<uint2*>(dst + db + (long long)c * dst_ld + r) = make_uint2(tile[2 * threadIdx.x][j], tile[2 * threadIdx.x + 1][j]);
  }
}

__global__ void __launch_bounds__(256) transpose16_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, int R, int C,
                                                         long long dst_ld, long long src_bs, long long dst_bs) {
  pdl_prologue();
  __shared__ uint32_t tile[64][33];                   // 64 rows of 64 16-bit values (32 words) + 1 word of padding
  const long long sb = (long long)blockIdx.z * src_bs, db = (long long)blockIdx.z * dst_bs;
  const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
#pragma unroll
  for (int j = threadIdx.y; j < 64; j += 8) {
    const int r = r0 + j, c = c0 + 2 * threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = *reinterpret_cast<const uint32_t*>(src + sb + (long long)r * C + c);
  }
  __syncthreads();
  // output row c (64 of them), pairs of r: words of two source rows, the same half of each
#pragma unroll
  for (int j = threadIdx.y; j < 64; j += 8) {
    const int c = c0 + j, r = r0 + 2 * threadIdx.x;
    if (c < C && r < R) {
      const uint32_t w0 = tile[2 * threadIdx.x][j >> 1], w1 = tile[2 * threadIdx.x + 1][j >> 1];
      const uint32_t lo = (j & 1) ? (w0 >> 16) : (w0 & 0xFFFFu), hi = (j & 1) ? (w1 >> 16) : (w1 & 0xFFFFu);
      *reinterpret_cast<uint32_t*>(dst + db + (long long)c * dst_ld + r) = lo | (hi << 16);
    }
  }
}

// 2-byte elements, 128 x 128 tiles: 256 contiguous bytes per row on both sides. The tile sits in shared memory as
// 32-bit words (pairs along c) with the word column XOR-ed by (row / 4): both the row-wise stores and the reads of
// four consecutive rows at one column are free of bank conflicts. R, C and the leading dimensions multiples of 4.
__global__ void __launch_bounds__(256) transpose16x4_kernel(uint16_t* __restrict__ dst, const uint16_t* __restrict__ src, int R, int C,
                                                           long long dst_ld, long long src_bs, long long dst_bs) {
  pdl_prologue();
  __shared__ uint32_t tile[128][64];
  const long long sb = (long long)blockIdx.z * src_bs, db = (long long)blockIdx.z * dst_bs;
  const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
  uint2 v[16];
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    const int r = r0 + threadIdx.y + 8 * q, c = c0 + 4 * threadIdx.x;
    v[q] = make_uint2(0, 0);
    if (r < R && c < C) v[q] = *reinterpret_cast<const uint2*>(src + sb + (long long)r * C + c);
  }
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    const int rl = threadIdx.y + 8 * q, k = (rl >> 2) & 31;
    tile[rl][(2 * threadIdx.x) ^ k] = v[q].x;
    tile[rl][(2 * threadIdx.x + 1) ^ k] = v[q].y;
  }
  __syncthreads();
  // output row c, four consecutive r per thread: the same half of one word column of four tile rows
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    const int j = threadIdx.y + 8 * q, c = c0 + j, r = r0 + 4 * threadIdx.x;
    if (c < C && r < R) {
      const int k = threadIdx.x & 31, w = (j >> 1) ^ k, sh = (j & 1) * 16;
      const uint32_t e0 = (tile[4 * threadIdx.x][w] >> sh) & 0xFFFFu, e1 = (tile[4 * threadIdx.x + 1][w] >> sh) & 0xFFFFu;
      const uint32_t e2 = (tile[4 * threadIdx.x + 2][w] >> sh) & 0xFFFFu, e3 = (tile[4 * threadIdx.x + 3][w] >> sh) & 0xFFFFu;
      *reinterpret_cast<uint2*>(dst + db + (long long)c * dst_ld + r) = make_uint2(e0 | (e1 << 16), e2 | (e3 << 16));
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Skinny products (M <= 8).
struct GemvParams {
  int M, N, K, G;
  long long a_ms, a_ks, a_gs, b_ld, b_gs;      // b_ld: stride of k (nc) or of n (kc)
  int kc, splits, c_kind, vec;                 // vec: 128-bit loads of B are aligned
  int b_static;                                // B may be read before the wait for the kernel in front
};

template <bool BF16>
__device__ __forceinline__ float lo16(uint32_t w) {
  if (BF16) return __uint_as_float(w << 16);
  return __half2float(__ushort_as_half((unsigned short)(w & 0xFFFFu)));
}
template <bool BF16>
__device__ __forceinline__ float hi16(uint32_t w) {
  if (BF16) return __uint_as_float(w & 0xFFFF0000u);
  return __half2float(__ushort_as_half((unsigned short)(w >> 16)));
}
template <bool BF16>
__device__ __forceinline__ float one16(uint16_t h) { return lo16<BF16>((uint32_t)h); }

// A[m][k0 .. k0 + len) of M rows -> dst[m][pad] as fp32 (zero past `len`), by 16-byte loads issued four at a time per
// thread when the rows allow it (k contiguous, 16-byte aligned starts): a loop of dependent scalar loads costs one
// memory round trip per iteration, which is what a skinny product's time is made of.
template <bool BF16>
__device__ __forceinline__ void stage_a_f32(float* __restrict__ dst, const uint16_t* __restrict__ Ag, int M, int rows, int pad,
                                            int len, long long a_ms, long long a_ks, int k0, int tid) {
  const bool wide = a_ks == 1 && (a_ms & 7) == 0 && (k0 & 7) == 0 && ((((uintptr_t)Ag) & 15) == 0) && (pad & 7) == 0;
  if (wide) {
    const int cpr = pad >> 3, chunks = rows * cpr;     // 8-element chunks per staged row
    for (int i0 = tid; i0 < chunks; i0 += 256 * 4) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + 256 * u;
        v[u] = make_uint4(0, 0, 0, 0);
        if (i < chunks) {
          const int m = i / cpr, c = i - m * cpr;
          if (m < M && 8 * c + 8 <= len) v[u] = *reinterpret_cast<const uint4*>(Ag + m * a_ms + k0 + 8 * c);
          else if (m < M && 8 * c < len) {
            uint32_t w[4] = {0, 0, 0, 0};
            for (int q = 0; q < 8 && 8 * c + q < len; ++q) w[q >> 1] |= (uint32_t)Ag[m * a_ms + k0 + 8 * c + q] << (16 * (q & 1));
            v[u] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + 256 * u;
        if (i < chunks) {
          float* d = dst + 8 * i;
          d[0] = lo16<BF16>(v[u].x); d[1] = hi16<BF16>(v[u].x); d[2] = lo16<BF16>(v[u].y); d[3] = hi16<BF16>(v[u].y);
          d[4] = lo16<BF16>(v[u].z); d[5] = hi16<BF16>(v[u].z); d[6] = lo16<BF16>(v[u].w); d[7] = hi16<BF16>(v[u].w);
        }
      }
    }
  } else {
    for (int i = tid; i < rows * pad; i += 256) {
      const int m = i / pad, kk = i - m * pad;
      dst[i] = (m < M && kk < len) ? one16<BF16>(Ag[m * a_ms + (long long)(k0 + kk) * a_ks]) : 0.f;
    }
  }
}

__device__ __forceinline__ void store_c(void* C, long long i, float v, int c_kind) {
  if (c_kind == 2) ((float*)C)[i] = v;
  else ((uint16_t*)C)[i] = (uint16_t)to16(v, c_kind);
}

// n contiguous in B. Grid (column panels of 256, K splits, groups), 256 threads: lane l of every warp owns the eight
// columns panel * 256 + 8 l .. + 7, warp w the rows k = kbeg + w, w + 8, ... of the CTA's K range; UNROLL rows are in
// flight per thread. The eight warps' sums meet in shared memory; with several K splits each CTA leaves its sums in
// `scratch` and the last one to arrive at the panel's counter adds the splits in order 0 .. S-1 (so the result does
// not depend on which CTA came last), stores the result and leaves the counter at zero for the next launch.
template <int MAXM, bool BF16, int UNROLL>
__global__ void __launch_bounds__(256) gemv16_nc_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ B,
                                                       void* __restrict__ C, float* __restrict__ scratch,
                                                       int* __restrict__ counters, GemvParams p) {
  extern __shared__ float gemv_smem[];
  float* a_s = gemv_smem;                              // [MAXM][kc_pad]
  const int kc_pad = p.kc + 8 * UNROLL;
  float* red = a_s + MAXM * kc_pad;                    // [8 warps][MAXM][256]
  __shared__ int is_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int panel = blockIdx.x, sp = blockIdx.y, g = blockIdx.z;
  const int kbeg = sp * p.kc, kend = min(p.K, kbeg + p.kc);
  const uint16_t* Ag = A + (long long)g * p.a_gs;
  const uint16_t* Bg = B + (long long)g * p.b_gs;
  const int n = panel * 256 + lane * 8;
  const bool vec = p.vec && n + 8 <= p.N;
  uint4 v[UNROLL];
  auto load_rows = [&](int k) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int kk = k + 8 * u;
      v[u] = make_uint4(0, 0, 0, 0);
      if (kk < kend) {
        const uint16_t* src = Bg + (long long)kk * p.b_ld + n;
        if (vec) v[u] = __ldcs(reinterpret_cast<const uint4*>(src));
        else if (n < p.N) {
          uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (n + j < p.N) w[j >> 1] |= (uint32_t)src[j] << (16 * (j & 1));
          v[u] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  };
  // The first rows of B are on their way before the slice of A is staged; when nothing in flight writes B they are
  // requested even before the wait for the kernel in front, whose tail then overlaps the first HBM round trip.
  if (p.b_static) load_rows(kbeg + warp);
  pdl_prologue();
  if (!p.b_static) load_rows(kbeg + warp);
  stage_a_f32<BF16>(a_s, Ag, p.M, MAXM, kc_pad, kend - kbeg, p.a_ms, p.a_ks, kbeg, tid);
  __syncthreads();
  float acc[MAXM][8];
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[m][j] = 0.f;
  for (int k = kbeg + warp; k < kend; k += 8 * UNROLL) {
    if (k != kbeg + warp) load_rows(k);
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const float b0 = lo16<BF16>(v[u].x), b1 = hi16<BF16>(v[u].x), b2 = lo16<BF16>(v[u].y), b3 = hi16<BF16>(v[u].y);
      const float b4 = lo16<BF16>(v[u].z), b5 = hi16<BF16>(v[u].z), b6 = lo16<BF16>(v[u].w), b7 = hi16<BF16>(v[u].w);
      const int kk = k + 8 * u - kbeg;                 // rows past kend read the zero padding of a_s
#pragma unroll
      for (int m = 0; m < MAXM; ++m) {
        const float a = a_s[m * kc_pad + kk];
        acc[m][0] = fmaf(a, b0, acc[m][0]); acc[m][1] = fmaf(a, b1, acc[m][1]);
        acc[m][2] = fmaf(a, b2, acc[m][2]); acc[m][3] = fmaf(a, b3, acc[m][3]);
        acc[m][4] = fmaf(a, b4, acc[m][4]); acc[m][5] = fmaf(a, b5, acc[m][5]);
        acc[m][6] = fmaf(a, b6, acc[m][6]); acc[m][7] = fmaf(a, b7, acc[m][7]);
      }
    }
  }
  // the eight warps' sums of all M rows meet in shared memory at once: thread t finishes column t of every row
  const int nn = panel * 256 + tid;
  __syncthreads();
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int j = 0; j < 8; ++j) red[(warp * MAXM + m) * 256 + lane * 8 + j] = acc[m][j];
  __syncthreads();
  float fin[MAXM];
#pragma unroll
  for (int m = 0; m < MAXM; ++m) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[(w * MAXM + m) * 256 + tid];
    fin[m] = s;
  }
  if (nn < p.N) {
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
      if (m >= p.M) break;
      if (p.splits == 1) store_c(C, ((long long)g * p.M + m) * p.N + nn, fin[m], p.c_kind);
      else scratch[(((long long)g * p.splits + sp) * p.M + m) * p.N + nn] = fin[m];
    }
  }
  if (p.splits == 1) return;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    int* ctr = counters + g * gridDim.x + panel;
    const int old = atomicAdd(ctr, 1);
    is_last = old == p.splits - 1;
    if (is_last) *ctr = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // The last CTA to arrive adds the splits: warp w takes the splits w, w + 8, ... for the eight columns of each of its
  // lanes and every row (independent loads, several in flight), then the eight warps' sums are added in warp order: a
  // fixed order whichever CTA came last.
  const bool vec4 = (p.N & 3) == 0;
  float t[MAXM][8];
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int j = 0; j < 8; ++j) t[m][j] = 0.f;
#pragma unroll 2
  for (int q = warp; q < p.splits; q += 8) {
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
      if (m >= p.M) break;
      const float* src = scratch + (((long long)g * p.splits + q) * p.M + m) * p.N + n;
      if (vec4 && n + 8 <= p.N) {
        const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src)), v1 = __ldcg(reinterpret_cast<const float4*>(src) + 1);
        t[m][0] += v0.x; t[m][1] += v0.y; t[m][2] += v0.z; t[m][3] += v0.w;
        t[m][4] += v1.x; t[m][5] += v1.y; t[m][6] += v1.z; t[m][7] += v1.w;
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (n + j < p.N) t[m][j] += __ldcg(src + j);
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int j = 0; j < 8; ++j) red[(warp * MAXM + m) * 256 + lane * 8 + j] = t[m][j];
  __syncthreads();
  if (nn < p.N) {
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
      if (m >= p.M) break;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[(w * MAXM + m) * 256 + tid];
      store_c(C, ((long long)g * p.M + m) * p.N + nn, s, p.c_kind);
    }
  }
}

// n contiguous in B, a small B (probabilities against a value cache: a few hundred rows of a few hundred columns). The
// whole product is one round trip to memory: a CTA owns 32 columns and all of K, its 64 groups of four lanes take the
// rows k = slot, slot + 64, ... (up to 16 independent 16-byte loads per lane, all issued before any is used), the
// sums of the groups meet by warp shuffles and once through shared memory in warp order. No K split across CTAs, so no
// scratch, no counter and no second pass.
template <int MAXM, bool BF16>
__global__ void __launch_bounds__(256) gemv16_nc_small_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ B,
                                                             void* __restrict__ C, GemvParams p) {
  constexpr int R = 16;
  extern __shared__ float gemv_smem[];
  float* a_s = gemv_smem;                              // [MAXM][K]
  float* red = a_s + MAXM * p.K;                       // [8 warps][MAXM][32]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.y, cg = lane & 3, slot = warp * 8 + (lane >> 2);
  const uint16_t* Ag = A + (long long)g * p.a_gs;
  const uint16_t* Bg = B + (long long)g * p.b_gs;
  const int n = blockIdx.x * 32 + cg * 8;
  const bool vec = p.vec && n + 8 <= p.N;
  uint4 v[R];
  auto load_rows = [&]() {
#pragma unroll
    for (int j = 0; j < R; ++j) {
      const int k = slot + 64 * j;
      v[j] = make_uint4(0, 0, 0, 0);
      if (k < p.K) {
        const uint16_t* src = Bg + (long long)k * p.b_ld + n;
        if (vec) v[j] = *reinterpret_cast<const uint4*>(src);
        else if (n < p.N) {
          uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (n + q < p.N) w[q >> 1] |= (uint32_t)src[q] << (16 * (q & 1));
          v[j] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }
  };
  if (p.b_static) load_rows();
  pdl_prologue();
  if (!p.b_static) load_rows();
  stage_a_f32<BF16>(a_s, Ag, p.M, MAXM, p.K, p.K, p.a_ms, p.a_ks, 0, tid);
  __syncthreads();
  float acc[MAXM][8];
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int q = 0; q < 8; ++q) acc[m][q] = 0.f;
#pragma unroll
  for (int j = 0; j < R; ++j) {
    const int k = slot + 64 * j;
    if (k >= p.K) break;
    const float b0 = lo16<BF16>(v[j].x), b1 = hi16<BF16>(v[j].x), b2 = lo16<BF16>(v[j].y), b3 = hi16<BF16>(v[j].y);
    const float b4 = lo16<BF16>(v[j].z), b5 = hi16<BF16>(v[j].z), b6 = lo16<BF16>(v[j].w), b7 = hi16<BF16>(v[j].w);
#pragma unroll
    for (int m = 0; m < MAXM; ++m) {
      const float a = a_s[m * p.K + k];
      acc[m][0] = fmaf(a, b0, acc[m][0]); acc[m][1] = fmaf(a, b1, acc[m][1]);
      acc[m][2] = fmaf(a, b2, acc[m][2]); acc[m][3] = fmaf(a, b3, acc[m][3]);
      acc[m][4] = fmaf(a, b4, acc[m][4]); acc[m][5] = fmaf(a, b5, acc[m][5]);
      acc[m][6] = fmaf(a, b6, acc[m][6]); acc[m][7] = fmaf(a, b7, acc[m][7]);
    }
  }
  // the eight row slots of a warp (lanes with equal lane & 3) by shuffles, then the eight warps in warp order
#pragma unroll
  for (int m = 0; m < MAXM; ++m)
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float s = acc[m][q];
      s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
      s += __shfl_xor_sync(0xFFFFFFFFu, s, 8);
      s += __shfl_xor_sync(0xFFFFFFFFu, s, 16);
      if (lane < 4) red[(warp * MAXM + m) * 32 + cg * 8 + q] = s;
    }
  __syncthreads();
  for (int t = tid; t < MAXM * 32; t += 256) {
    const int m = t >> 5, c = t & 31, nn = blockIdx.x * 32 + c;
    if (m < p.M && nn < p.N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[(w * MAXM + m) * 32 + c];
      store_c(C, ((long long)g * p.M + m) * p.N + nn, s, p.c_kind);
    }
  }
}

// k contiguous in B (a tied-embedding logits product, scores against a key cache, a weight transposed in front of a
// decode loop). Grid (CTAs, groups), 256 threads; a warp takes NW output columns at a time, its lanes stride over k with
// 128-bit loads (K a multiple of 8), A sits in shared memory as 16-bit values, per-lane sums meet in a warp-shuffle tree.
template <int MAXM, bool BF16, int NW>
__global__ void __launch_bounds__(256) gemv16_kc_kernel(const uint16_t* __restrict__ A, const uint16_t* __restrict__ B,
                                                       void* __restrict__ C, GemvParams p) {
  extern __shared__ float gemv_smem[];
  uint16_t* a_s = (uint16_t*)gemv_smem;                // [M][K], 16-byte aligned rows (K % 8 == 0)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.y;
  const uint16_t* Ag = A + (long long)g * p.a_gs;
  const uint16_t* Bg = B + (long long)g * p.b_gs;
  // UNR chunks of 8 k per column are loaded before any is used: NW * UNR independent 16-byte loads in flight per lane
  constexpr int UNR = NW == 1 ? 8 : 2;
  const int tasks = (p.N + NW - 1) / NW;
  uint4 b[UNR][NW];
  auto load_cols = [&](int n0, int k0) {
#pragma unroll
    for (int u = 0; u < UNR; ++u)
#pragma unroll
      for (int q = 0; q < NW; ++q) {
        const int k = k0 + 256 * u;
        b[u][q] = (n0 + q < p.N && k < p.K) ? __ldcs(reinterpret_cast<const uint4*>(Bg + (long long)(n0 + q) * p.b_ld + k))
                                            : make_uint4(0, 0, 0, 0);
      }
  };
  // The warp's first loads of B are on their way before A is staged; when nothing in flight writes B they are requested
  // even before the wait for the kernel in front, whose tail then overlaps the first HBM round trip.
  const int first_task = blockIdx.x * 8 + warp;
  if (p.b_static && first_task < tasks) load_cols(first_task * NW, lane * 8);
  pdl_prologue();
  if (!p.b_static && first_task < tasks) load_cols(first_task * NW, lane * 8);
  if (p.a_ks == 1 && (p.a_ms & 7) == 0 && (p.a_gs & 7) == 0 && (((uintptr_t)A) & 15) == 0) {
    const int chunks = p.K >> 3;                        // rows of A are whole 16-byte chunks (K % 8 == 0)
    for (int i0 = tid; i0 < p.M * chunks; i0 += 256 * 4) {
      uint4 v[4];                                       // four loads in flight per thread
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + 256 * u;
        if (i < p.M * chunks) {
          const int m = i / chunks, c = i - m * chunks;
          v[u] = *reinterpret_cast<const uint4*>(Ag + m * p.a_ms + 8 * c);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + 256 * u;
        if (i < p.M * chunks) reinterpret_cast<uint4*>(a_s)[i] = v[u];
      }
    }
  } else {
    for (int i = tid; i < p.M * p.K; i += 256) {
      const int m = i / p.K, k = i % p.K;
      a_s[i] = Ag[m * p.a_ms + (long long)k * p.a_ks];
    }
  }
  __syncthreads();
  for (int task = first_task; task < tasks; task += gridDim.x * 8) {
    const int n0 = task * NW;
    float acc[NW][MAXM];
#pragma unroll
    for (int q = 0; q < NW; ++q)
#pragma unroll
      for (int m = 0; m < MAXM; ++m) acc[q][m] = 0.f;
    for (int k0 = lane * 8; k0 < p.K; k0 += 256 * UNR) {
      if (task != first_task || k0 != lane * 8) load_cols(n0, k0);
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const int k = k0 + 256 * u;
        if (k >= p.K) break;
#pragma unroll
        for (int m = 0; m < MAXM; ++m) {
          if (m >= p.M) break;
          const uint4 a = *reinterpret_cast<const uint4*>(a_s + m * p.K + k);
          const float a0 = lo16<BF16>(a.x), a1 = hi16<BF16>(a.x), a2 = lo16<BF16>(a.y), a3 = hi16<BF16>(a.y);
          const float a4 = lo16<BF16>(a.z), a5 = hi16<BF16>(a.z), a6 = lo16<BF16>(a.w), a7 = hi16<BF16>(a.w);
#pragma unroll
          for (int q = 0; q < NW; ++q) {
            float s = acc[q][m];
            s = fmaf(a0, lo16<BF16>(b[u][q].x), s); s = fmaf(a1, hi16<BF16>(b[u][q].x), s);
            s = fmaf(a2, lo16<BF16>(b[u][q].y), s); s = fmaf(a3, hi16<BF16>(b[u][q].y), s);
            s = fmaf(a4, lo16<BF16>(b[u][q].z), s); s = fmaf(a5, hi16<BF16>(b[u][q].z), s);
            s = fmaf(a6, lo16<BF16>(b[u][q].w), s); s = fmaf(a7, hi16<BF16>(b[u][q].w), s);
            acc[q][m] = s;
          }
        }
      }
    }
#pragma unroll
    for (int q = 0; q < NW; ++q)
#pragma unroll
      for (int m = 0; m < MAXM; ++m) {
        float s = acc[q][m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (lane == 0 && m < p.M && n0 + q < p.N) store_c(C, ((long long)g * p.M + m) * p.N + n0 + q, s, p.c_kind);
      }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &st) == cudaSuccess &&
        st == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)f;
  });
  return fn;
}

// Rank-3 map over a strided matrix per group: dimension 0 is the contiguous one (`inner` elements), dimension 1
// has `outer` rows `ld` elements apart, dimension 2 the groups `gs` elements apart.
bool make_map(CUtensorMap* map, const void* base, int in_fmt, long long inner, long long outer, long long groups, long long ld,
              long long gs, int box_inner, int box_outer) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return false;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)groups};
  // a stride of a dimension of extent 1 is never used but must still be a multiple of 16 bytes
  cuuint64_t strides[2] = {(cuuint64_t)(outer > 1 ? ld : inner + ((8 - inner % 8) % 8)) * 2,
                           (cuuint64_t)(groups > 1 ? gs : 8) * 2};
  if (strides[0] % 16 || strides[1] % 16) return false;
  cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, in_fmt == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void*)base, dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

// Tiled tensor map with the 128-byte swizzle over this GPU's memory: `kind` 0 f16, 1 bf16, 2 f32; dims[0] is the
// contiguous dimension; strides (bytes) belong to dims[1..]. False when the driver refuses (alignment, extents).
bool encode_tensor_map(void* map, int kind, int rank, const void* base, const unsigned long long* dims,
                       const unsigned long long* strides_bytes, const unsigned* box) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc || rank < 1 || rank > 5) return false;
  cuuint64_t d[5], st[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; i++) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; if (i + 1 < rank) st[i] = strides_bytes[i]; }
  const CUtensorMapDataType dt = kind == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : (kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  return enc((CUtensorMap*)map, dt, (cuuint32_t)rank, (void*)base, d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

}  // namespace

bool gemm16_plan(Gemm16Launch& g, bool aligned) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.G <= 0) return false;
  g.scratch_floats = 0;
  g.counters = 0;
  g.split_k = 1;
  const int SMS = 148;
  if (g.M <= 8) {
    if (g.b_ns == 1 && g.K <= 1024 && (long long)g.K * g.N <= (1 << 20)) {
      g.path = 3;                                    // a small B: one round trip, no K split across CTAs
      return true;
    }
    if (g.b_ns == 1) {
      // every element of B once: column panels of 256 times K splits should give each SM several CTAs
      g.path = 1;
      const int panels = (g.N + 255) / 256;
      // one wave of CTAs (four of these CTAs fit an SM), each with at least 64 rows of K
      long long want = ((long long)SMS * 4) / ((long long)panels * g.G);
      want = std::max<long long>(1, std::min<long long>(want, (g.K + 63) / 64));
      int kc = (int)((g.K + want - 1) / want);
      kc = (kc + 7) / 8 * 8;
      kc = std::min(kc, g.M == 1 ? 2048 : 512);      // the K range's slice of A (fp32) shares shared memory with the sums
      g.gemv_kc = kc;
      g.split_k = (g.K + kc - 1) / kc;
      if (g.split_k > 1) {
        g.scratch_floats = (long long)g.G * g.split_k * g.M * g.N;
        g.counters = g.G * panels;
      }
      return true;
    }
    if (g.b_ks == 1 && g.K % 8 == 0 && g.b_ns % 8 == 0 && g.b_gs % 8 == 0 && (long long)g.M * g.K * 2 <= 96 * 1024) {
      g.path = 2;
      g.nw = (long long)g.N * g.G >= (long long)SMS * 8 * 4 * 4 ? 4 : 1;
      return true;
    }
  }
  if (!aligned) return false;
  if (!((g.a_ks == 1 || g.a_ms == 1) && (g.b_ks == 1 || g.b_ns == 1))) return false;
  g.path = 0;
  const long long mt = (g.M + 127) / 128;
  const int ktiles = (g.K + 63) / 64;
  auto tiles_for = [&](int bn) { return mt * ((g.N + bn - 1) / bn) * g.G; };
  // Tile width and K split by a small cost model: cycles per 64-deep k-tile of a 128 x bn tile (a 256-wide tile is
  // bound by the tensor pipe, narrower ones by the shared-memory reads of the MMA unit), a fixed cost per tile, whole
  // waves of CTAs over the SMs, and for a split the pass that adds the partial sums (a launch plus its traffic). A split
  // is considered only while it fits one wave and leaves each CTA four k-tiles. Ties go to the wider tile, then to the
  // smaller split.
  {
    double best = 1e30;
    int best_split = 1;
    for (int bn : {256, 128, 64}) {
      if (bn > 64 && g.N <= bn / 2) continue;
      const double per_kt = bn == 256 ? 512.0 : (bn == 128 ? 256.0 : 192.0);
      const long long t = tiles_for(bn);
      for (int split = 1; split <= 16; ++split) {
        if (split > 1 && (t * split > SMS || ktiles / split < 4)) break;
        const int kps = (ktiles + split - 1) / split;
        const long long waves = (t * split + SMS - 1) / SMS;
        const double fill_kt = (128.0 + bn) * 64.0 * 2.0 / 90.0;            // one SM takes its tiles in at about 90 bytes per cycle
        double cost = (double)waves * (kps * std::max(per_kt, fill_kt) + 400.0);
        if (split > 1) cost += 2500.0 + (double)g.G * g.M * g.N * 4.0 * (split + 1) / 3000.0;     // second pass: launch + bytes at ~3 KB per cycle
        if (cost < best * 0.999) { best = cost; g.bn = bn; best_split = split; }
      }
    }
    g.kt_per_split = ktiles;
    if (best_split > 1) {
      g.kt_per_split = (ktiles + best_split - 1) / best_split;
      g.split_k = (ktiles + g.kt_per_split - 1) / g.kt_per_split;
      if (g.split_k > 1) g.scratch_floats = (long long)g.split_k * g.G * g.M * g.N;
      else g.kt_per_split = ktiles;
    }
  }
  return true;
}

cudaError_t launch_transpose2d(void* dst, const void* src, int elem_bytes, long long batch, long long rows, long long cols,
                               long long dst_ld, long long dst_batch_stride, cudaStream_t stream, int* launches) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return cudaSuccess;
  if (batch > 65535 || rows >= (1LL << 31) || cols >= (1LL << 31)) return cudaErrorInvalidValue;
  dim3 block(32, 8);
  if (elem_bytes == 4 && rows % 2 == 0 && cols % 2 == 0 && dst_ld % 2 == 0 && dst_batch_stride % 2 == 0 &&
      (((uintptr_t)dst | (uintptr_t)src) & 7) == 0 && !getenv("B200_NARROW_TRANSPOSE")) {
    dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64), (unsigned)batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    launch_k(transpose32x2_kernel, grid, block, 0, stream, (uint32_t*)dst, (const uint32_t*)src, (int)rows, (int)cols, dst_ld, rows * cols,
             dst_batch_stride);
  } else if (elem_bytes == 4) {
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    launch_k(transpose32_kernel, grid, block, 0, stream, (uint32_t*)dst, (const uint32_t*)src, (int)rows, (int)cols, dst_ld, rows * cols,
                                                   dst_batch_stride);
  } else if (elem_bytes == 2 && rows % 4 == 0 && cols % 4 == 0 && dst_ld % 4 == 0 && dst_batch_stride % 4 == 0 &&
             (((uintptr_t)dst | (uintptr_t)src) & 7) == 0 && !getenv("B200_NARROW_TRANSPOSE")) {
    dim3 grid((unsigned)((cols + 127) / 128), (unsigned)((rows + 127) / 128), (unsigned)batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    launch_k(transpose16x4_kernel, grid, block, 0, stream, (uint16_t*)dst, (const uint16_t*)src, (int)rows, (int)cols, dst_ld, rows * cols,
             dst_batch_stride);
  } else if (elem_bytes == 2 && rows % 2 == 0 && cols % 2 == 0 && dst_ld % 2 == 0 && dst_batch_stride % 2 == 0 &&
             (((uintptr_t)dst | (uintptr_t)src) & 3) == 0) {
    dim3 grid((unsigned)((cols + 63) / 64), (unsigned)((rows + 63) / 64), (unsigned)batch);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    launch_k(transpose16_kernel, grid, block, 0, stream, (uint16_t*)dst, (const uint16_t*)src, (int)rows, (int)cols, dst_ld, rows * cols,
                                                   dst_batch_stride);
  } else {
    return cudaErrorInvalidValue;
  }
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_repack_rows16(void* dst, const void* src, long long rows, long long cols, long long dst_ld, long long src_ld,
                                 cudaStream_t stream, int* launches) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (rows > 65535) {
    // the row index rides in gridDim.y: longer matrices go out in slabs
    for (long long r0 = 0; r0 < rows; r0 += 65535) {
      const long long nr = std::min<long long>(65535, rows - r0);
      cudaError_t e = launch_repack_rows16((uint16_t*)dst + r0 * dst_ld, (const uint16_t*)src + r0 * src_ld, nr, cols, dst_ld,
                                           src_ld, stream, launches);
      if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
  }
  dim3 grid((unsigned)std::min<long long>(64, (cols + 255) / 256), (unsigned)rows);
  launch_k(repack_rows16_kernel, grid, 256, 0, stream, (uint16_t*)dst, (const uint16_t*)src, rows, cols, dst_ld, src_ld);
  if (launches) (*launches)++;
  return cudaGetLastError();
}

cudaError_t launch_gemm16(const Gemm16Launch& g, const void* A, const void* B, void* C, float* scratch, int* counters,
                          int* error_flag, cudaStream_t stream, int* launches, const char** why) {
  *why = nullptr;
  const bool bf16 = g.in_fmt == 1;
  if (g.path == 1 || g.path == 2 || g.path == 3) {
    GemvParams p;
    p.M = g.M; p.N = g.N; p.K = g.K; p.G = g.G;
    p.a_ms = g.a_ms; p.a_ks = g.a_ks; p.a_gs = g.a_gs;
    p.b_ld = g.path == 2 ? g.b_ns : g.b_ks;
    p.b_gs = g.b_gs;
    p.kc = g.gemv_kc; p.splits = g.split_k; p.c_kind = g.c_kind;
    p.vec = (((uintptr_t)B) & 15) == 0 && p.b_ld % 8 == 0 && g.b_gs % 8 == 0;
    p.b_static = g.b_static;
    const int maxm = g.M == 1 ? 1 : 8;
    if (g.path == 3) {
      dim3 grid((g.N + 31) / 32, g.G);
      const size_t smem = (size_t)maxm * g.K * 4 + (size_t)8 * maxm * 32 * 4;
      if (maxm == 1 && bf16) launch_k(gemv16_nc_small_kernel<1, true>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, p);
      else if (maxm == 1) launch_k(gemv16_nc_small_kernel<1, false>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, p);
      else if (bf16) launch_k(gemv16_nc_small_kernel<8, true>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, p);
      else launch_k(gemv16_nc_small_kernel<8, false>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, p);
    } else if (g.path == 1) {
      if (g.split_k > 1 && (!scratch || !counters)) { *why = "skinny product without its scratch"; return cudaErrorInvalidValue; }
      dim3 grid((g.N + 255) / 256, g.split_k, g.G);
      static bool configured[64] = {};
      if (first_use_on_this_device(configured)) {
        cudaFuncSetAttribute(gemv16_nc_kernel<8, true, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * (2048 + 32) * 4 + 65536);
        cudaFuncSetAttribute(gemv16_nc_kernel<8, false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 8 * (2048 + 32) * 4 + 65536);
      }
      const int unroll = maxm == 1 ? 8 : 4;
      const size_t smem = (size_t)maxm * (g.gemv_kc + 8 * unroll) * 4 + (size_t)maxm * 8 * 256 * 4;
      if (maxm == 1 && bf16) launch_k(gemv16_nc_kernel<1, true, 8>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, scratch, counters, p);
      else if (maxm == 1) launch_k(gemv16_nc_kernel<1, false, 8>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, scratch, counters, p);
      else if (bf16) launch_k(gemv16_nc_kernel<8, true, 4>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, scratch, counters, p);
      else launch_k(gemv16_nc_kernel<8, false, 4>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, scratch, counters, p);
    } else {
      if (!p.vec) { *why = "skinny product: B is not 16-byte aligned"; return cudaErrorInvalidValue; }
      static bool configured[64] = {};
      if (first_use_on_this_device(configured)) {
#define SETKC(MM, BF, NW_) cudaFuncSetAttribute(gemv16_kc_kernel<MM, BF, NW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)
        SETKC(1, true, 1); SETKC(1, true, 4); SETKC(1, false, 1); SETKC(1, false, 4);
        SETKC(8, true, 1); SETKC(8, true, 4); SETKC(8, false, 1); SETKC(8, false, 4);
#undef SETKC
      }
      const int tasks = (g.N + g.nw - 1) / g.nw;
      dim3 grid((unsigned)std::max(1, std::min((tasks + 7) / 8, sm_count() * 8)), g.G);
      const size_t smem = (size_t)g.M * g.K * 2;
#define LAUNCHKC(MM, BF, NW_) launch_k(gemv16_kc_kernel<MM, BF, NW_>, grid, 256, smem, stream, (const uint16_t*)A, (const uint16_t*)B, C, p)
      if (maxm == 1) {
        if (bf16) { if (g.nw == 4) LAUNCHKC(1, true, 4); else LAUNCHKC(1, true, 1); }
        else { if (g.nw == 4) LAUNCHKC(1, false, 4); else LAUNCHKC(1, false, 1); }
      } else {
        if (bf16) { if (g.nw == 4) LAUNCHKC(8, true, 4); else LAUNCHKC(8, true, 1); }
        else { if (g.nw == 4) LAUNCHKC(8, false, 4); else LAUNCHKC(8, false, 1); }
      }
#undef LAUNCHKC
    }
    if (launches) (*launches)++;
    return cudaGetLastError();
  }

  // tensor-core tiles
  Gemm16Params p;
  p.M = g.M; p.N = g.N; p.K = g.K; p.G = g.G;
  p.a_mn = g.a_ks == 1 ? 0 : 1;
  p.b_mn = g.b_ks == 1 ? 0 : 1;
  if (g.K == 1) { p.a_mn = g.a_ms == 1 ? 1 : 0; p.b_mn = g.b_ns == 1 ? 1 : 0; }
  p.split_k = g.split_k; p.kt_per_split = g.kt_per_split;
  p.in_fmt = g.in_fmt; p.c_kind = g.c_kind;
  p.mtiles = (g.M + G_BM - 1) / G_BM;
  p.ntiles = (g.N + g.bn - 1) / g.bn;
  if (g.split_k > 1 && !scratch) { *why = "split product without its scratch"; return cudaErrorInvalidValue; }
  alignas(64) CUtensorMap tm_a, tm_b;
  bool ok;
  if (!p.a_mn) ok = make_map(&tm_a, A, g.in_fmt, g.K, g.M, g.G, g.a_ms, g.a_gs, 64, 128);
  else ok = make_map(&tm_a, A, g.in_fmt, g.M, g.K, g.G, g.a_ks, g.a_gs, 64, 64);
  if (ok) {
    if (!p.b_mn) ok = make_map(&tm_b, B, g.in_fmt, g.K, g.N, g.G, g.b_ns, g.b_gs, 64, g.bn);
    else ok = make_map(&tm_b, B, g.in_fmt, g.N, g.K, g.G, g.b_ks, g.b_gs, 64, 64);
  }
  if (!ok) { *why = "cuTensorMapEncodeTiled refused an operand (alignment or extent)"; return cudaErrorInvalidValue; }
  static bool configured[64] = {};
  if (first_use_on_this_device(configured)) {
    cudaFuncSetAttribute(gemm16_tma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, G16Cfg<64>::SMEM);
    cudaFuncSetAttribute(gemm16_tma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, G16Cfg<128>::SMEM);
    cudaFuncSetAttribute(gemm16_tma_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, G16Cfg<256>::SMEM);
  }
  const long long tiles = (long long)p.mtiles * p.ntiles * p.G * p.split_k;
  const unsigned grid = (unsigned)std::min<long long>(tiles, sm_count());
  if (g.bn == 256) launch_k(gemm16_tma_kernel<256>, grid, G_THREADS, G16Cfg<256>::SMEM, stream, tm_a, tm_b, C, scratch, error_flag, p);
  else if (g.bn == 128) launch_k(gemm16_tma_kernel<128>, grid, G_THREADS, G16Cfg<128>::SMEM, stream, tm_a, tm_b, C, scratch, error_flag, p);
  else launch_k(gemm16_tma_kernel<64>, grid, G_THREADS, G16Cfg<64>::SMEM, stream, tm_a, tm_b, C, scratch, error_flag, p);
  if (launches) (*launches)++;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  if (g.split_k > 1) {
    const long long total = (long long)g.G * g.M * g.N;
    launch_k(splitk_sum16_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, scratch, C, total, g.split_k, g.c_kind);
    if (launches) (*launches)++;
    e = cudaGetLastError();
  }
  return e;
}

void set_programmatic_launch(bool on) { g_programmatic_launch = on; }

}  // namespace b200
