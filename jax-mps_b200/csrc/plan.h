// Kernel plan: what a compiled StableHLO program looks like to the executor.
//
// The reference replays a traced MLX graph op by op
// (src/pjrt_plugin/mlx_executable.cc:699-725, 799-1008). Here compilation
// produces a static plan: every tensor that must exist in memory has a slot
// (argument, constant, arena offset or result), and every step is one kernel
// launch (a generated fused kernel, the implicit-GEMM kernel, a copy), a
// control-flow construct over nested plans, or a collective.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

#include "gemm16.h"
#include "ir.h"

namespace b200 {

struct Slot {
  enum Kind { ARG, CONST, TEMP, RESULT } kind = TEMP;
  size_t bytes = 0;
  int index = -1;          // ARG: argument number; RESULT: result number; CONST: constant number
  int arena = 0;           // TEMP: which arena
  size_t offset = 0;       // TEMP: byte offset in the arena
  TensorType type;
};

// Parameters of the implicit-GEMM kernel (convolution and dot_general share it).
// C[g][m][n] = sum_k A(g, m, k) * B(g, k, n); A is gathered through a row
// table (one entry per m) and a column table (one entry per k).
struct IGemmParams {
  int M = 0, N = 0, K = 0, groups = 1;
  // A element: a_row[m].off + a_col[k].off + (ih / ldh) * a_sh + (iw / ldw) * a_sw, valid when
  // ih = a_row[m].h0 + a_col[k].dh and iw likewise are in [0, Hd) x [0, Wd) and divisible by ldh / ldw.
  int Hd = 1, Wd = 1, ldh = 1, ldw = 1;
  long long a_sh = 0, a_sw = 0;
  long long a_gs = 0, b_gs = 0, c_gs = 0;    // group strides (elements)
  long long b_sn = 1, c_sn = 1;              // stride of n in B and C
  int a_contig = 0;                          // 0: k contiguous in A, 1: m contiguous
  int b_contig = 0;                          // 0: n contiguous in B, 1: k contiguous
  int split_k = 1;
  int needs_mask = 0;
  int vec = 0;                               // both operands gather in uniform, aligned 16-byte chunks
  int kt_stride = 0;                         // > 0: the last igemm arg is a table [m-tile][1 + kt_stride] of k-tiles to visit
  int seg = 0;                               // vec, and aligned runs of 32 along the contiguous dimensions are uniform
  int c_vec = 0;                             // consecutive n are consecutive floats in C (2: and rows start on multiples of four floats)
  // A operand of a stride-1 convolution over a dense NHWC input whose 128-row tiles are whole output rows: every
  // k-tile of A is one box of the input (32 channels x OW pixels x rows x images at one filter tap), fetched by a
  // single TMA tiled copy with zero fill outside the image instead of a table-driven gather.
  int a_tma = 0;
  int tma_c = 0, tma_w = 0, tma_h = 0, tma_n = 0;        // input extents (channels, width, height, images)
  int tma_ow = 0, tma_oh = 0, tma_box_h = 0, tma_box_n = 0;
  int tma_kw = 0, tma_pad_h = 0, tma_pad_w = 0, tma_rdil_h = 1, tma_rdil_w = 1;
};

struct Plan;

// Row scatter (kernels.cu): ints of scratch and kernel launches for `updates` updates into `rows` rows.
long long scatter_rows_scratch_ints(long long rows, long long updates);
int scatter_rows_launches(long long rows, long long updates);
long long scatter_elems_scratch_ints(long long updates);
int scatter_elems_launches(long long numel);

struct Step {
  enum Kind { KERNEL, IGEMM, MEMCPY, MEMSET, WHILE, CASE, ALL_REDUCE, SCATTER, JOIN, GEMM16, REPACK16, TRANSPOSE, ALL_GATHER } kind = KERNEL;
  std::string label;                  // op names, for profiling and error text
  // KERNEL
  int kernel = -1;                    // index into Executable::kernels
  unsigned grid[3] = {1, 1, 1}, block[3] = {1, 1, 1};
  std::vector<int> args;              // slot ids, in kernel-parameter order
  int n_outs = 0;                     // KERNEL: the first n_outs args are written, the rest only read
  // IGEMM: args = {A, B, C, a_row, a_col, b_row(k), b_col(n), c_row(m), c_col(n), a_grp, b_grp, c_grp, [split-K scratch]}
  IGemmParams ig;
  // GEMM16: args = {A, B, C, [fp32 scratch], [counters]}; iparams = {has scratch, has counters}
  // REPACK16: args = {dst, src}; iparams = {rows, cols, dst_ld, src_ld}
  // TRANSPOSE: args = {dst, src}; iparams = {element bytes, batch, rows, cols, dst_ld, dst batch stride, dst offset (elements)}
  Gemm16Launch g16;
  // MEMCPY: args = {dst, src}; MEMSET: args = {dst}
  size_t bytes = 0;
  // WHILE: sub[0] = cond, sub[1] = body; state/init/next slot lists; pred slot
  // CASE: sub = branches; args = {index}; branch_results[b][i] copied to results[i]
  std::vector<std::unique_ptr<Plan>> sub;
  std::vector<int> state, init, next;
  std::vector<char> swap;             // WHILE: per carried value, exchange the state and next pointers instead of copying
  std::vector<std::vector<int>> branch_results;
  std::vector<int> results;
  int pred = -1;
  long long trip_count = -1;          // statically known trip count of a counted loop
  // ALL_REDUCE: args = {in, out}; overlapped = issued on the collective stream, the next JOIN step makes the
  // compute stream wait for it
  bool overlapped = false;
  DT dtype = DT::F32;
  // ALL_GATHER: args = {in, out, [staging]}; bytes = operand bytes; iparams = {rows before all_gather_dim, bytes per such row}
  // SCATTER: args = {operand, indices, updates, result, scratch...}
  std::vector<long long> iparams;
};

struct Plan {
  std::vector<Step> steps;
  int arena = 0;                      // arena holding this plan's temporaries
};

struct KernelSource {
  std::string name;
  std::string body;                   // full __global__ definition
};

struct ConstData {
  std::vector<uint8_t> bytes;
};

struct ResultInfo {
  TensorType type;
  int slot = -1;
  int donated_arg = -1;               // argument whose storage this result may take over
};

struct CompiledProgram {
  std::string name;
  std::string fingerprint;
  std::vector<Slot> slots;
  std::vector<ConstData> consts;
  std::vector<KernelSource> kernels;
  std::vector<size_t> arena_bytes;
  Plan main;
  std::vector<TensorType> arg_types;
  std::vector<ResultInfo> results;
  int num_partitions = 1, num_replicas = 1;
  int launches_per_execute = -1;      // static count when the plan has no data-dependent control flow
  std::string dump;                   // human-readable plan (B200_DUMP_PLAN)
};

struct CompileOptions {
  bool fuse = true;                   // B200_NO_FUSE=1 turns fusion off (one kernel per op)
  int num_partitions = 1;
  int partition_id = 0;               // this process's partition (stablehlo.partition_id)
};

// StableHLO module -> plan. Throws CompileError (unsupported op, malformed attribute...).
std::unique_ptr<CompiledProgram> compile_module(Module& m, const CompileOptions& opts);

// The device-function library every generated kernel is compiled with.
const char* codegen_prelude();

}  // namespace b200
