// CUDA source generation for fused kernels.
//
// A fused kernel evaluates a DAG of StableHLO operations per output element.
// Every value is computed "in a context": an index tuple into its own shape.
// Elementwise operations pass the context through; broadcast, transpose,
// reshape, reverse, slice, pad, concatenate, dynamic_slice and
// dynamic_update_slice rewrite it for their operand(s); values that are not
// part of the fusion are loaded from memory at the context's position.
// The reference gets the same effect from mlx::core::compile
// (src/pjrt_plugin/mlx_executable.cc:882); here the composition is printed
// as straight-line CUDA over the device functions of the prelude.
#pragma once
#include <functional>
#include <map>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "ir.h"

namespace b200 {

const char* c_type(DT d);        // register type
const char* s_type(DT d);        // storage type
std::string literal(DT d, const uint8_t* bytes);

struct Ctx {
  std::vector<std::string> idx;   // one index expression per dimension (may be empty until needed)
  std::string lin;                // row-major linear index expression, when known
  std::vector<int64_t> shape;
};

class Emitter {
 public:
  std::function<bool(Op*)> is_internal;        // op evaluated inline (fusion member or duplicable)
  std::string idx_t = "int";
  std::vector<Value*> inputs;                  // external values, in parameter order
  std::map<Value*, std::string> bound;         // values bound to a fixed expression (region arguments)
  bool round_small_floats = true;              // round bf16/f16 results after every op
  std::string name_prefix;                     // keeps variable names of cooperating emitters apart

  std::string emit(Value* v, Ctx c);
  std::string input_name(Value* v);
  void seed_inputs(const std::vector<Value*>& vs) { for (Value* v : vs) input_name(v); }   // fix the first parameters
  void line(const std::string& s);
  std::string fresh(const char* prefix);
  void ensure_idx(Ctx& c);
  std::string lin_of(Ctx& c);
  void push_scope() { memo_.emplace_back(); indent_ += 2; }
  void pop_scope() { memo_.pop_back(); indent_ -= 2; }
  std::string str() const { return os_.str(); }
  // Evaluates a region whose operations are all scalar elementwise ops.
  std::vector<std::string> emit_scalar_region(Block* b, const std::vector<std::string>& args);
  int indent_ = 4;

 private:
  std::string elementwise(Op* op, const std::vector<std::string>& a);
  std::string load(Value* v, Ctx& c);
  std::string key(Value* v, Ctx& c);
  std::ostringstream os_;
  std::vector<std::map<std::string, std::string>> memo_{1};
  std::map<Value*, int> in_index_;
  int nvar_ = 0;
};

bool is_elementwise_op(const std::string& short_name);

}  // namespace b200
