// Launch description of a 16-bit floating-point contraction, shared by the plan compiler (which sizes the scratch
// memory from it) and the kernel launcher (which follows it). The kernels are described in kernels.h / gemm16.cu.
#pragma once

namespace b200 {
struct Gemm16Launch {
  int M = 0, N = 0, K = 0, G = 1;
  long long a_ms = 0, a_ks = 0, a_gs = 0;   // element strides of m, k and the group in A
  long long b_ks = 0, b_ns = 0, b_gs = 0;   // element strides of k, n and the group in B
  int in_fmt = 1;                           // operands: 0 f16, 1 bf16
  int c_kind = 1;                           // result: 0 f16, 1 bf16, 2 f32
  int b_static = 0;                         // B is not written by the kernel in front of this one (a program input, or made
                                            // in front of the loop whose body this product belongs to): the skinny
                                            // kernels may fetch it before they wait for that kernel
  // filled by gemm16_plan (the compiler sizes the scratch from it, the launcher follows it)
  int path = 0, bn = 128, split_k = 1, kt_per_split = 0, gemv_kc = 0, nw = 1;
  long long scratch_floats = 0;             // fp32 partial sums
  int counters = 0;                         // zero-initialised ints (path 1 with splits; the kernel leaves them at zero)
};

// Chooses kernel, tile width and K split for a contraction; false when no 16-bit kernel applies (the caller then
// widens the operands to f32). `aligned`: bases and non-unit strides are multiples of 16 bytes.
bool gemm16_plan(Gemm16Launch& g, bool aligned);

}  // namespace b200
