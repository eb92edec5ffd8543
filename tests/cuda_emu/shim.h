// Just enough of the CUDA execution model to run the plan compiler's generated kernels on host threads: one OS
// thread per CUDA thread of a block, blocks one after the other. Block and warp barriers let a thread that has
// returned drop out, as exited CUDA threads do. Test infrastructure: nothing in the product includes this file.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

using std::isfinite;
template <typename T> static inline T max(T a, T b) { return a < b ? b : a; }
template <typename T> static inline T min(T a, T b) { return b < a ? b : a; }
using std::isnan;
using std::isinf;
using std::signbit;

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline __attribute__((always_inline))
#define __launch_bounds__(...)
#define __shared__ static
#define __align__(n) __attribute__((aligned(n)))

struct alignas(8) uint2 { unsigned x, y; };
struct alignas(16) uint4 { unsigned x, y, z, w; };
struct alignas(8) float2 { float x, y; };
struct alignas(16) float4 { float x, y, z, w; };
static inline uint2 make_uint2(unsigned x, unsigned y) { return {x, y}; }
static inline uint4 make_uint4(unsigned x, unsigned y, unsigned z, unsigned w) { return {x, y, z, w}; }
static inline float2 make_float2(float x, float y) { return {x, y}; }
static inline float4 make_float4(float x, float y, float z, float w) { return {x, y, z, w}; }

namespace emu {
struct Dim { unsigned x = 1, y = 1, z = 1; };
extern thread_local Dim t_thread, t_block;
extern thread_local int t_lane;
extern Dim g_block_dim, g_grid_dim;
// implemented by the runner (runner.cc), which owns the threads and their barriers
void block_barrier();
void warp_barrier();
unsigned long long warp_exchange(unsigned long long value, int source_lane);     // value of source_lane, own value if out of range
unsigned warp_ballot(int pred);
int warp_lanes();
}  // namespace emu

#define threadIdx emu::t_thread
#define blockIdx emu::t_block
#define blockDim emu::g_block_dim
#define gridDim emu::g_grid_dim

static inline void __syncthreads() { emu::block_barrier(); }
static inline void __syncwarp(unsigned = 0xFFFFFFFFu) { emu::warp_barrier(); }
static inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
static inline void __threadfence_block() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

template <typename T>
static inline T emu_exchange(T v, int src) {
  unsigned long long raw = 0;
  std::memcpy(&raw, &v, sizeof(T));
  const unsigned long long got = emu::warp_exchange(raw, src);
  T r;
  std::memcpy(&r, &got, sizeof(T));
  return r;
}
template <typename T> static inline T __shfl_sync(unsigned, T v, int src) { return emu_exchange(v, src & 31); }
template <typename T> static inline T __shfl_xor_sync(unsigned, T v, int m) { return emu_exchange(v, emu::t_lane ^ m); }
template <typename T> static inline T __shfl_down_sync(unsigned, T v, unsigned d) { return emu_exchange(v, emu::t_lane + (int)d < 32 ? emu::t_lane + (int)d : emu::t_lane); }
template <typename T> static inline T __shfl_up_sync(unsigned, T v, unsigned d) { return emu_exchange(v, emu::t_lane - (int)d >= 0 ? emu::t_lane - (int)d : emu::t_lane); }
static inline unsigned __ballot_sync(unsigned, int pred) { return emu::warp_ballot(pred); }
static inline int __all_sync(unsigned m, int pred) { return __ballot_sync(m, pred) == (emu::warp_lanes() == 32 ? 0xFFFFFFFFu : ((1u << emu::warp_lanes()) - 1u)); }
static inline int __any_sync(unsigned m, int pred) { return __ballot_sync(m, pred) != 0; }

static inline float __uint_as_float(unsigned u) { float f; std::memcpy(&f, &u, 4); return f; }
static inline float __int_as_float(int u) { float f; std::memcpy(&f, &u, 4); return f; }
static inline unsigned __float_as_uint(float f) { unsigned u; std::memcpy(&u, &f, 4); return u; }
static inline int __float_as_int(float f) { int u; std::memcpy(&u, &f, 4); return u; }
static inline long long __double_as_longlong(double f) { long long u; std::memcpy(&u, &f, 8); return u; }
static inline double __longlong_as_double(long long u) { double f; std::memcpy(&f, &u, 8); return f; }
static inline unsigned __umulhi(unsigned a, unsigned b) { return (unsigned)(((unsigned long long)a * b) >> 32); }
static inline int __popc(unsigned a) { return __builtin_popcount(a); }
static inline int __popcll(unsigned long long a) { return __builtin_popcountll(a); }
static inline int __clz(int a) { return a == 0 ? 32 : __builtin_clz((unsigned)a); }
static inline int __clzll(long long a) { return a == 0 ? 64 : __builtin_clzll((unsigned long long)a); }
template <typename T> static inline T __ldcg(const T* p) { return *(const volatile T*)p; }
template <> inline float4 __ldcg<float4>(const float4* p) { float4 r; std::memcpy(&r, (const void*)p, sizeof r); return r; }
template <> inline uint4 __ldcg<uint4>(const uint4* p) { uint4 r; std::memcpy(&r, (const void*)p, sizeof r); return r; }
template <typename T> static inline T __ldg(const T* p) { return *p; }
static inline int atomicAdd(int* p, int v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline unsigned atomicAdd(unsigned* p, unsigned v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline unsigned long long atomicAdd(unsigned long long* p, unsigned long long v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline float atomicAdd(float* p, float v) {
  unsigned* u = (unsigned*)p;
  unsigned old = __atomic_load_n(u, __ATOMIC_SEQ_CST);
  while (true) {
    const unsigned want = __float_as_uint(__uint_as_float(old) + v);
    if (__atomic_compare_exchange_n(u, &old, want, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST)) return __uint_as_float(old);
  }
}
static inline float rsqrtf(float x) { return 1.0f / sqrtf(x); }
static inline double rsqrt(double x) { return 1.0 / sqrt(x); }
// inverse error function by Newton steps on erf (the library gives erf to full precision)
static inline double erfinv(double y) {
  if (!(y > -1.0 && y < 1.0)) return y == 1.0 ? INFINITY : (y == -1.0 ? -INFINITY : NAN);
  double w = -log((1.0 - y) * (1.0 + y)), x;
  if (w < 5.0) { w -= 2.5; x = 2.81022636e-08; x = 3.43273939e-07 + x * w; x = -3.5233877e-06 + x * w; x = -4.39150654e-06 + x * w; x = 0.00021858087 + x * w; x = -0.00125372503 + x * w; x = -0.00417768164 + x * w; x = 0.246640727 + x * w; x = 1.50140941 + x * w; }
  else { w = sqrt(w) - 3.0; x = -0.000200214257; x = 0.000100950558 + x * w; x = 0.00134934322 + x * w; x = -0.00367342844 + x * w; x = 0.00573950773 + x * w; x = -0.0076224613 + x * w; x = 0.00943887047 + x * w; x = 1.00167406 + x * w; x = 2.83297682 + x * w; }
  x *= y;
  for (int k = 0; k < 3; k++) x -= (erf(x) - y) / (1.1283791670955126 * exp(-x * x));
  return x;
}
static inline float erfinvf(float y) { return (float)erfinv((double)y); }

extern "C" void emu_launch(void* fn, int nargs, void** args, int gx, int gy, int gz, int bx, int by, int bz);
