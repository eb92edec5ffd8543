// In-memory form of a StableHLO module and the text reader that builds it.
//
// The reference hands the program to MLIR (src/pjrt_plugin/stablehlo_parser.cc:
// 187-285); this plugin owns its front end: a recursive-descent reader of MLIR
// text (generic operation form, plus the custom assembly of the common
// StableHLO operations) producing a flat SSA graph with nested regions.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace b200 {

enum class DT : uint8_t { INVALID = 0, PRED, I8, I16, I32, I64, U8, U16, U32, U64, F16, BF16, F32, F64, TOKEN };

inline size_t dt_size(DT d) {
  switch (d) {
    case DT::PRED: case DT::I8: case DT::U8: return 1;
    case DT::I16: case DT::U16: case DT::F16: case DT::BF16: return 2;
    case DT::I32: case DT::U32: case DT::F32: return 4;
    case DT::I64: case DT::U64: case DT::F64: return 8;
    default: return 0;
  }
}
inline bool dt_is_float(DT d) { return d == DT::F16 || d == DT::BF16 || d == DT::F32 || d == DT::F64; }
inline bool dt_is_signed(DT d) { return d == DT::I8 || d == DT::I16 || d == DT::I32 || d == DT::I64; }
inline bool dt_is_unsigned(DT d) { return d == DT::U8 || d == DT::U16 || d == DT::U32 || d == DT::U64; }
inline bool dt_is_int(DT d) { return dt_is_signed(d) || dt_is_unsigned(d); }
const char* dt_name(DT d);          // MLIR spelling: f32, bf16, i32, ui32, i1
DT dt_from_name(const std::string& s);

struct CompileError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct TensorType {
  DT dt = DT::INVALID;
  std::vector<int64_t> dims;
  int64_t numel() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
  size_t bytes() const { return (size_t)numel() * dt_size(dt); }
  int rank() const { return (int)dims.size(); }
  bool operator==(const TensorType& o) const { return dt == o.dt && dims == o.dims; }
  std::string str() const;
};

struct Op;
struct Block;

struct Value {
  int id = -1;
  TensorType type;
  Op* def = nullptr;        // null for block arguments
  int def_index = 0;
  Block* owner = nullptr;   // block whose argument this is (def == nullptr)
  int arg_index = -1;
  std::string name;
  std::vector<Op*> users;   // filled by Module::link_users
};

struct Block {
  std::vector<Value*> args;
  std::vector<std::unique_ptr<Op>> ops;
  Op* parent_op = nullptr;
};

struct Op {
  std::string name;                               // e.g. "stablehlo.add"
  std::vector<Value*> operands;
  std::vector<Value*> results;
  std::map<std::string, std::string> attrs;       // raw attribute text, decoded on demand
  std::vector<std::unique_ptr<Block>> regions;
  Block* parent = nullptr;
  int pos = -1;                                   // position in the flattened schedule

  bool is(const char* n) const { return name == n; }
  std::string short_name() const {
    auto p = name.find('.');
    return p == std::string::npos ? name : name.substr(p + 1);
  }
  bool has(const std::string& k) const { return attrs.count(k) != 0; }
  const std::string& attr(const std::string& k) const;
};

struct Func {
  std::string name;
  bool is_private = false;
  std::unique_ptr<Block> body;
  std::vector<TensorType> result_types;
  std::vector<std::map<std::string, std::string>> arg_attrs;
};

struct Module {
  std::string name;
  std::map<std::string, std::string> attrs;
  std::map<std::string, std::unique_ptr<Func>> funcs;
  std::deque<Value> values;     // stable addresses

  Value* new_value(const TensorType& t, const std::string& name = "");
  Func* main() const;
};

// Parses MLIR text. Throws CompileError with a position on malformed input.
std::unique_ptr<Module> parse_module(const char* text, size_t size);

// ---- attribute decoding (raw text -> values) -------------------------------
int64_t attr_int(const std::string& raw);
bool attr_bool(const std::string& raw);
std::vector<int64_t> attr_i64s(const std::string& raw);         // array<i64: ..>, dense<..>, [..]
std::string attr_str(const std::string& raw);                   // strips quotes
std::string attr_enum(const std::string& raw);                  // '#stablehlo<x GT>' -> GT
std::map<std::string, std::vector<int64_t>> attr_struct(const std::string& raw);   // '#stablehlo.dot<a = [..], b = 1>'
// 'dense<..> : tensor<..>' -> raw little-endian bytes of the full tensor
// (pred as one byte per element) and whether every element is equal.
struct DenseValue {
  TensorType type;
  std::vector<uint8_t> data;
  bool splat = false;
};
DenseValue attr_dense(const std::string& raw);
TensorType parse_type(const std::string& text);

uint16_t f32_to_bf16(float f);
float bf16_to_f32(uint16_t h);
uint16_t f32_to_f16(float f);
float f16_to_f32(uint16_t h);

}  // namespace b200
