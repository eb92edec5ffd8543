// Device-side helpers shared by the tensor-core kernels (kernels.cu, gemm16.cu): shared-memory addresses,
// mbarriers with bounded waits, the K-major shared-memory matrix descriptor and single-lane election.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace b200 {
namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Bounded wait: false when the phase did not complete within the budget.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// First statement of a kernel that may be launched with programmatic stream serialization: the kernel is scheduled
// while the one in front of it drains, and waits here until everything in front of it has completed and its memory
// is visible. Without the launch attribute this is a no-op. (Letting dependents start earlier still, with
// griddepcontrol.launch_dependents, lost time on the measured programs: 6.42 -> 6.73 ms on the DistilBERT-shaped step.)
__device__ __forceinline__ void pdl_prologue() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), LBO unused (1), descriptor version 1
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// One lane of a converged warp. The MMA warps run their loops with all 32 lanes (so that descriptor arithmetic
// stays warp-uniform) and only the elected lane issues tcgen05.mma / tcgen05.commit: issued from a loop that a
// single thread runs alone, the same instruction stream feeds the tensor core at two thirds of the rate.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// cudaFuncSetAttribute applies to the current device: a process that drives several GPUs configures each of them once.
static bool first_use_on_this_device(bool (&done)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
  if (done[dev]) return false;
  done[dev] = true;
  return true;
}

}  // namespace
}  // namespace b200
