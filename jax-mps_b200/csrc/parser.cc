// MLIR text reader for StableHLO modules (see ir.h).
//
// Generic form is the canonical input:
//   %r = "stablehlo.op"(%a, %b) <{props}> ({regions}) {attrs} : (types) -> types
// The custom assembly of the operations that occur in the reference's own
// raw-MLIR test (tests/test_ops.py:216-269) and in typical jax lowerings is
// accepted too and normalised to the same Op structure.
#include <cmath>
#include <cstring>
#include <set>
#include <sstream>

#include "ir.h"

namespace b200 {

const char* dt_name(DT d) {
  switch (d) {
    case DT::PRED: return "i1";
    case DT::I8: return "i8";
    case DT::I16: return "i16";
    case DT::I32: return "i32";
    case DT::I64: return "i64";
    case DT::U8: return "ui8";
    case DT::U16: return "ui16";
    case DT::U32: return "ui32";
    case DT::U64: return "ui64";
    case DT::F16: return "f16";
    case DT::BF16: return "bf16";
    case DT::F32: return "f32";
    case DT::F64: return "f64";
    case DT::TOKEN: return "token";
    default: return "invalid";
  }
}

DT dt_from_name(const std::string& s) {
  static const std::map<std::string, DT> m = {
      {"i1", DT::PRED}, {"i8", DT::I8},   {"i16", DT::I16},   {"i32", DT::I32},   {"i64", DT::I64},
      {"ui8", DT::U8},  {"ui16", DT::U16}, {"ui32", DT::U32},  {"ui64", DT::U64},  {"f16", DT::F16},
      {"bf16", DT::BF16}, {"f32", DT::F32}, {"f64", DT::F64},  {"u8", DT::U8},     {"u16", DT::U16},
      {"u32", DT::U32},  {"u64", DT::U64}};
  auto it = m.find(s);
  if (it == m.end()) throw CompileError("unsupported element type '" + s + "'");
  return it->second;
}

std::string TensorType::str() const {
  if (dt == DT::TOKEN) return "!stablehlo.token";
  std::string s = "tensor<";
  for (auto d : dims) s += std::to_string(d) + "x";
  return s + dt_name(dt) + ">";
}

const std::string& Op::attr(const std::string& k) const {
  auto it = attrs.find(k);
  if (it == attrs.end()) throw CompileError(name + ": missing attribute '" + k + "'");
  return it->second;
}

Value* Module::new_value(const TensorType& t, const std::string& name) {
  values.emplace_back();
  Value* v = &values.back();
  v->id = (int)values.size() - 1;
  v->type = t;
  v->name = name;
  return v;
}

Func* Module::main() const {
  auto it = funcs.find("main");
  if (it != funcs.end()) return it->second.get();
  for (auto& kv : funcs)
    if (!kv.second->is_private) return kv.second.get();
  throw CompileError("module has no entry function 'main'");
}

uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t f32_to_f16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    int shift = 14 - exp;
    uint32_t r = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (r & 1))) r++;
    return (uint16_t)(sign | r);
  }
  uint32_t r = ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) r++;
  return (uint16_t)(sign | r);
}
float f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FFu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { man <<= 1; e++; } while (!(man & 0x400u));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
  else u = sign | ((exp - 15 + 127) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}

// ---------------------------------------------------------------------------
// scanner
// ---------------------------------------------------------------------------
namespace {

struct Scanner {
  const char* s;
  size_t n, i = 0;
  Scanner(const char* t, size_t len) : s(t), n(len) {}

  [[noreturn]] void fail(const std::string& what) const {
    size_t line = 1;
    for (size_t k = 0; k < i && k < n; k++) line += s[k] == '\n';
    std::string ctx(s + i, std::min<size_t>(60, n - i));
    throw CompileError("MLIR parse error (line " + std::to_string(line) + "): " + what + " near '" + ctx + "'");
  }
  void ws() {
    while (i < n) {
      char c = s[i];
      if (c == ' ' || c == '\t' || c == '\r' || c == '\n') i++;
      else if (c == '/' && i + 1 < n && s[i + 1] == '/') {
        while (i < n && s[i] != '\n') i++;
      } else break;
    }
  }
  bool peek(const char* lit) {
    ws();
    size_t l = strlen(lit);
    return i + l <= n && strncmp(s + i, lit, l) == 0;
  }
  bool accept(const char* lit) {
    if (peek(lit)) { i += strlen(lit); return true; }
    return false;
  }
  void expect(const char* lit) {
    if (!accept(lit)) fail(std::string("expected '") + lit + "'");
  }
  static bool idc(char c) { return isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$'; }
  std::string ident() {
    ws();
    size_t j = i;
    while (j < n && idc(s[j])) j++;
    if (j == i) fail("expected identifier");
    std::string r(s + i, j - i);
    i = j;
    return r;
  }
  std::string ssa() {
    ws();
    if (i >= n || s[i] != '%') fail("expected SSA value");
    size_t j = i + 1;
    while (j < n && (idc(s[j]) || s[j] == '#' || s[j] == '-')) j++;
    std::string r(s + i, j - i);
    i = j;
    return r;
  }
  int64_t integer() {
    ws();
    size_t j = i;
    if (j < n && (s[j] == '-' || s[j] == '+')) j++;
    while (j < n && isdigit((unsigned char)s[j])) j++;
    if (j == i) fail("expected integer");
    int64_t v = strtoll(std::string(s + i, j - i).c_str(), nullptr, 10);
    i = j;
    return v;
  }
  std::string string_lit() {
    ws();
    if (i >= n || s[i] != '"') fail("expected string");
    size_t j = i + 1;
    std::string out;
    while (j < n && s[j] != '"') {
      if (s[j] == '\\' && j + 1 < n) { out += s[j + 1]; j += 2; }
      else out += s[j++];
    }
    i = j + 1;
    return out;
  }
  // Raw text up to the first top-level character in `stops`.
  std::string balanced(const char* stops) {
    ws();
    int depth = 0;
    size_t j = i;
    while (j < n) {
      char c = s[j];
      if (c == '"') {
        j++;
        while (j < n && s[j] != '"') j += (s[j] == '\\') ? 2 : 1;
      } else if (c == '(' || c == '[' || c == '{' || c == '<') depth++;
      else if (c == ')' || c == ']' || c == '}' || c == '>') {
        if (depth == 0 && strchr(stops, c)) break;
        if (!(c == '>' && j > 0 && s[j - 1] == '-')) depth--;
      } else if (depth == 0 && strchr(stops, c)) break;
      j++;
    }
    size_t a = i, b = j;
    while (b > a && isspace((unsigned char)s[b - 1])) b--;
    i = j;
    return std::string(s + a, b - a);
  }
};

TensorType read_type(Scanner& sc) {
  TensorType t;
  if (sc.accept("tensor<")) {
    while (true) {
      size_t j = sc.i;
      while (j < sc.n && isdigit((unsigned char)sc.s[j])) j++;
      if (j > sc.i && j < sc.n && sc.s[j] == 'x') {
        t.dims.push_back(strtoll(std::string(sc.s + sc.i, j - sc.i).c_str(), nullptr, 10));
        sc.i = j + 1;
      } else break;
    }
    if (sc.peek("?")) sc.fail("dynamic shapes are not supported");
    t.dt = dt_from_name(sc.ident());
    sc.expect(">");
    return t;
  }
  if (sc.accept("!stablehlo.token")) { t.dt = DT::TOKEN; return t; }
  sc.fail("expected tensor type");
}

std::vector<TensorType> read_type_list(Scanner& sc) {
  std::vector<TensorType> out;
  if (sc.accept("(")) {
    if (!sc.accept(")")) {
      do { out.push_back(read_type(sc)); } while (sc.accept(","));
      sc.expect(")");
    }
  } else out.push_back(read_type(sc));
  return out;
}

void read_attr_dict(Scanner& sc, const char* close, std::map<std::string, std::string>& out) {
  if (sc.accept(close)) return;
  std::string stops = std::string(",") + close[0];
  do {
    sc.ws();
    std::string key = (sc.i < sc.n && sc.s[sc.i] == '"') ? sc.string_lit() : sc.ident();
    if (sc.accept("=")) out[key] = sc.balanced(stops.c_str());
    else out[key] = "unit";
  } while (sc.accept(","));
  sc.expect(close);
}

void skip_loc(Scanner& sc) {
  if (sc.accept("loc(")) { sc.balanced(")"); sc.expect(")"); }
}

const std::set<std::string>& same_type_ops() {
  static const std::set<std::string> s = {
      "add", "subtract", "multiply", "divide", "maximum", "minimum", "power", "remainder", "atan2", "and", "or",
      "xor", "shift_left", "shift_right_logical", "shift_right_arithmetic", "exponential", "log", "sqrt", "rsqrt",
      "negate", "abs", "floor", "ceil", "sine", "cosine", "tanh", "tan", "logistic", "sign", "log_plus_one",
      "exponential_minus_one", "cbrt", "not", "popcnt", "count_leading_zeros", "round_nearest_even",
      "round_nearest_afz", "clamp"};
  return s;
}

struct ModuleParser {
  Scanner sc;
  Module* m;
  // scope stack of SSA names
  std::vector<std::map<std::string, Value*>> scopes;

  ModuleParser(const char* t, size_t n, Module* mod) : sc(t, n), m(mod) {}

  Value* lookup(const std::string& name) {
    for (auto it = scopes.rbegin(); it != scopes.rend(); ++it) {
      auto f = it->find(name);
      if (f != it->end()) return f->second;
    }
    sc.fail("use of undefined value " + name);
  }
  void define(const std::string& name, Value* v) { scopes.back()[name] = v; }

  // "#loc3 = loc(...)" lines that a module printed with debug information carries in front of or behind it
  void skip_location_aliases() {
    while (sc.peek("#loc")) {
      sc.balanced("\n");
    }
  }

  void parse() {
    bool wrapped = false;
    skip_location_aliases();
    if (sc.accept("module")) {
      wrapped = true;
      if (sc.accept("@")) m->name = sc.ident();
      if (sc.accept("attributes")) { sc.expect("{"); read_attr_dict(sc, "}", m->attrs); }
      sc.expect("{");
    }
    while (sc.peek("func.func")) func();
    if (wrapped) sc.expect("}");
    skip_loc(sc);
    skip_location_aliases();
    sc.ws();
    if (sc.i != sc.n) sc.fail("unexpected trailing text");
  }

  void func() {
    sc.expect("func.func");
    auto f = std::make_unique<Func>();
    if (sc.accept("private")) f->is_private = true;
    else sc.accept("public");
    sc.expect("@");
    f->name = sc.ident();
    f->body = std::make_unique<Block>();
    scopes.emplace_back();
    sc.expect("(");
    if (!sc.accept(")")) {
      do {
        std::string n = sc.ssa();
        sc.expect(":");
        TensorType t = read_type(sc);
        std::map<std::string, std::string> a;
        if (sc.accept("{")) read_attr_dict(sc, "}", a);
        skip_loc(sc);
        Value* v = m->new_value(t, n);
        v->owner = f->body.get();
        v->arg_index = (int)f->body->args.size();
        f->body->args.push_back(v);
        f->arg_attrs.push_back(a);
        define(n, v);
      } while (sc.accept(","));
      sc.expect(")");
    }
    if (sc.accept("->")) {
      if (sc.accept("(")) {
        if (!sc.accept(")")) {
          do {
            f->result_types.push_back(read_type(sc));
            if (sc.accept("{")) { std::map<std::string, std::string> a; read_attr_dict(sc, "}", a); }
          } while (sc.accept(","));
          sc.expect(")");
        }
      } else {
        f->result_types.push_back(read_type(sc));
      }
    }
    if (sc.accept("attributes")) { std::map<std::string, std::string> a; sc.expect("{"); read_attr_dict(sc, "}", a); }
    sc.expect("{");
    ops_until(f->body.get(), "}");
    sc.expect("}");
    skip_loc(sc);
    scopes.pop_back();
    m->funcs[f->name] = std::move(f);
  }

  void ops_until(Block* b, const char* close) {
    while (!sc.peek(close)) {
      auto op = parse_op();
      op->parent = b;
      b->ops.push_back(std::move(op));
    }
  }

  std::unique_ptr<Block> region(Op* parent) {
    sc.expect("{");
    auto b = std::make_unique<Block>();
    b->parent_op = parent;
    scopes.emplace_back();
    if (sc.accept("^")) {
      sc.ident();
      if (sc.accept("(")) {
        do {
          std::string n = sc.ssa();
          sc.expect(":");
          TensorType t = read_type(sc);
          skip_loc(sc);
          Value* v = m->new_value(t, n);
          v->owner = b.get();
          v->arg_index = (int)b->args.size();
          b->args.push_back(v);
          define(n, v);
        } while (sc.accept(","));
        sc.expect(")");
      }
      sc.expect(":");
    }
    ops_until(b.get(), "}");
    sc.expect("}");
    scopes.pop_back();
    return b;
  }

  void finish(Op* op, const std::vector<std::string>& names, const std::vector<TensorType>& types) {
    if (names.size() != types.size())
      sc.fail(op->name + ": " + std::to_string(names.size()) + " result names for " + std::to_string(types.size()) +
              " result types");
    for (size_t k = 0; k < names.size(); k++) {
      Value* v = m->new_value(types[k], names[k]);
      v->def = op;
      v->def_index = (int)k;
      op->results.push_back(v);
      define(names[k], v);
    }
  }

  std::unique_ptr<Op> parse_op() {
    sc.ws();
    std::vector<std::string> results;
    if (sc.i < sc.n && sc.s[sc.i] == '%') {
      do {
        std::string n = sc.ssa();
        if (sc.accept(":")) {
          int64_t k = sc.integer();
          for (int64_t j = 0; j < k; j++) results.push_back(n + "#" + std::to_string(j));
        } else results.push_back(n);
      } while (sc.accept(","));
      sc.expect("=");
    }
    sc.ws();
    auto op = std::make_unique<Op>();
    if (sc.i < sc.n && sc.s[sc.i] == '"') generic(op.get(), results);
    else pretty(op.get(), results);
    skip_loc(sc);
    return op;
  }

  void operand_list(Op* op, const char* close) {
    if (sc.accept(close)) return;
    do { op->operands.push_back(lookup(sc.ssa())); } while (sc.accept(","));
    sc.expect(close);
  }

  void generic(Op* op, const std::vector<std::string>& results) {
    op->name = sc.string_lit();
    sc.expect("(");
    operand_list(op, ")");
    if (sc.accept("<{")) read_attr_dict(sc, "}>", op->attrs);
    if (sc.peek("(")) {
      sc.expect("(");
      do {
        auto r = region(op);
        op->regions.push_back(std::move(r));
      } while (sc.accept(","));
      sc.expect(")");
    }
    if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
    sc.expect(":");
    read_type_list(sc);
    sc.expect("->");
    auto rts = read_type_list(sc);
    finish(op, results, rts);
  }

  std::string dims_attr() {   // "[1, 2]" -> "array<i64: 1, 2>"
    sc.expect("[");
    std::string d = sc.balanced("]");
    sc.expect("]");
    return d.empty() ? "array<i64>" : "array<i64: " + d + ">";
  }

  void pretty(Op* op, const std::vector<std::string>& results) {
    std::string name = sc.ident();
    std::string sh = name.rfind("stablehlo.", 0) == 0 ? name.substr(10) : name;
    op->name = name;
    if (name == "return" || name == "func.return" || name == "stablehlo.return") {
      op->name = name == "stablehlo.return" ? name : "func.return";
      if (sc.peek("%")) {
        do { op->operands.push_back(lookup(sc.ssa())); } while (sc.accept(","));
        sc.expect(":");
        do { read_type(sc); } while (sc.accept(","));
      }
      return;
    }
    if (sh == "constant") {
      std::string raw = sc.balanced("\n");
      // strip a trailing loc(...)
      auto lp = raw.rfind(" loc(");
      if (lp != std::string::npos) raw = raw.substr(0, lp);
      op->attrs["value"] = raw;
      auto c = raw.rfind(": ");
      if (c == std::string::npos) sc.fail("constant without type");
      finish(op, results, {parse_type(raw.substr(c + 2))});
      return;
    }
    if (same_type_ops().count(sh)) {
      do { op->operands.push_back(lookup(sc.ssa())); } while (sc.accept(","));
      if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
      sc.expect(":");
      if (sc.peek("(")) {          // (operand types) -> result type: clamp with scalar bounds
        read_type_list(sc);
        sc.expect("->");
        finish(op, results, read_type_list(sc));
        return;
      }
      TensorType t = read_type(sc);
      if (sc.accept(",")) {        // 'clamp'/'select'-style type lists or (..) -> .. forms
        do { t = read_type(sc); } while (sc.accept(","));
      }
      finish(op, results, {t});
      return;
    }
    if (sh == "composite") {
      op->attrs["name"] = "\"" + sc.string_lit() + "\"";
      while (sc.peek("%")) { op->operands.push_back(lookup(sc.ssa())); sc.accept(","); }
      if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "convert" || sh == "reshape" || sh == "bitcast_convert" || sh == "is_finite" ||
        sh == "optimization_barrier") {
      do { op->operands.push_back(lookup(sc.ssa())); } while (sc.accept(","));
      if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
      sc.expect(":");
      if (!sc.peek("(")) {
        // results typed like the operands: "convert %a : type" where nothing changes, "optimization_barrier %a, %b : t, t"
        std::vector<TensorType> ts;
        do { ts.push_back(read_type(sc)); } while (sc.accept(","));
        if (sc.accept("->")) ts = read_type_list(sc);
        finish(op, results, ts);
        return;
      }
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "compare") {
      std::string d = sc.ident();
      sc.expect(",");
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      op->operands.push_back(lookup(sc.ssa()));
      op->attrs["comparison_direction"] = "#stablehlo<comparison_direction " + d + ">";
      if (sc.accept(",")) op->attrs["compare_type"] = "#stablehlo<comparison_type " + sc.ident() + ">";
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "select") {
      do { op->operands.push_back(lookup(sc.ssa())); } while (sc.accept(","));
      sc.expect(":");
      TensorType t = read_type(sc);
      while (sc.accept(",")) t = read_type(sc);
      finish(op, results, {t});
      return;
    }
    if (sh == "broadcast_in_dim" || sh == "transpose") {
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      sc.expect("dims");
      sc.expect("=");
      op->attrs[sh == "transpose" ? "permutation" : "broadcast_dimensions"] = dims_attr();
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "iota") {
      sc.expect("dim");
      sc.expect("=");
      op->attrs["iota_dimension"] = std::to_string(sc.integer()) + " : i64";
      sc.expect(":");
      finish(op, results, {read_type(sc)});
      return;
    }
    if (sh == "concatenate") {
      while (sc.peek("%")) { op->operands.push_back(lookup(sc.ssa())); sc.expect(","); }
      sc.expect("dim");
      sc.expect("=");
      op->attrs["dimension"] = std::to_string(sc.integer()) + " : i64";
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "slice") {
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect("[");
      std::string st, li, sd;
      do {
        int64_t a = sc.integer();
        sc.expect(":");
        int64_t b = sc.integer();
        int64_t c = 1;
        if (sc.accept(":")) c = sc.integer();
        st += (st.empty() ? "" : ", ") + std::to_string(a);
        li += (li.empty() ? "" : ", ") + std::to_string(b);
        sd += (sd.empty() ? "" : ", ") + std::to_string(c);
      } while (sc.accept(","));
      sc.expect("]");
      op->attrs["start_indices"] = "array<i64: " + st + ">";
      op->attrs["limit_indices"] = "array<i64: " + li + ">";
      op->attrs["strides"] = "array<i64: " + sd + ">";
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "dynamic_slice" || sh == "dynamic_update_slice") {
      while (sc.peek("%")) {
        op->operands.push_back(lookup(sc.ssa()));
        if (!sc.accept(",")) break;
      }
      if (sc.accept("sizes")) { sc.expect("="); op->attrs["slice_sizes"] = dims_attr(); }
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "dot_general") {
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      op->operands.push_back(lookup(sc.ssa()));
      std::string lb = "[]", rb = "[]", lc = "[]", rc = "[]";
      while (sc.accept(",")) {
        std::string key = sc.ident();
        sc.expect("=");
        if (key == "precision") { sc.expect("["); sc.balanced("]"); sc.expect("]"); continue; }
        sc.expect("[");
        std::string a = "[" + sc.balanced("]") + "]";
        sc.expect("]");
        sc.expect("x");
        sc.expect("[");
        std::string b = "[" + sc.balanced("]") + "]";
        sc.expect("]");
        if (key == "batching_dims") { lb = a; rb = b; }
        else if (key == "contracting_dims") { lc = a; rc = b; }
        else sc.fail("dot_general: unknown clause " + key);
      }
      op->attrs["dot_dimension_numbers"] = "#stablehlo.dot<lhs_batching_dimensions = " + lb +
                                           ", rhs_batching_dimensions = " + rb + ", lhs_contracting_dimensions = " + lc +
                                           ", rhs_contracting_dimensions = " + rc + ">";
      if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (sh == "reduce") {
      // stablehlo.reduce(%a init: %i) applies stablehlo.add across dimensions = [1] : (..) -> ..
      sc.expect("(");
      std::vector<Value*> ins, inits;
      // several inputs are printed as (%a init: %i), (%b init: %j)
      while (true) {
        ins.push_back(lookup(sc.ssa()));
        sc.expect("init:");
        inits.push_back(lookup(sc.ssa()));
        if (sc.accept(",")) continue;                      // further pairs inside the same parentheses
        sc.expect(")");
        size_t save = sc.i;
        if (sc.accept(",") && sc.accept("(")) continue;    // the next pair in parentheses of its own
        sc.i = save;
        break;
      }
      op->operands = ins;
      op->operands.insert(op->operands.end(), inits.begin(), inits.end());
      if (sc.accept("applies")) {
        std::string body = sc.ident();
        sc.expect("across");
        sc.expect("dimensions");
        sc.expect("=");
        op->attrs["dimensions"] = dims_attr();
        sc.expect(":");
        read_type_list(sc);
        sc.expect("->");
        auto rts = read_type_list(sc);
        // synthesise the body
        auto b = std::make_unique<Block>();
        b->parent_op = op;
        TensorType st;
        st.dt = rts[0].dt;
        Value* a0 = m->new_value(st, "%acc");
        Value* a1 = m->new_value(st, "%val");
        for (Value* v : {a0, a1}) { v->owner = b.get(); v->arg_index = (int)b->args.size(); b->args.push_back(v); }
        auto inner = std::make_unique<Op>();
        inner->name = body;
        inner->operands = {a0, a1};
        inner->parent = b.get();
        Value* r = m->new_value(st, "%red");
        r->def = inner.get();
        inner->results.push_back(r);
        auto ret = std::make_unique<Op>();
        ret->name = "stablehlo.return";
        ret->operands = {r};
        ret->parent = b.get();
        b->ops.push_back(std::move(inner));
        b->ops.push_back(std::move(ret));
        op->regions.push_back(std::move(b));
        finish(op, results, rts);
        return;
      }
      sc.expect("across");
      sc.expect("dimensions");
      sc.expect("=");
      op->attrs["dimensions"] = dims_attr();
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      auto rts = read_type_list(sc);
      sc.expect("reducer");
      // reducer(%a: t, %b: t) (%c: t, %d: t) { ... }
      auto b = std::make_unique<Block>();
      b->parent_op = op;
      scopes.emplace_back();
      std::vector<std::pair<std::string, TensorType>> firsts, seconds;
      while (sc.accept("(")) {
        std::string n1 = sc.ssa(); sc.expect(":"); TensorType t1 = read_type(sc); sc.expect(",");
        std::string n2 = sc.ssa(); sc.expect(":"); TensorType t2 = read_type(sc); sc.expect(")");
        firsts.push_back({n1, t1});
        seconds.push_back({n2, t2});
      }
      for (auto* lst : {&firsts, &seconds})
        for (auto& p : *lst) {
          Value* v = m->new_value(p.second, p.first);
          v->owner = b.get();
          v->arg_index = (int)b->args.size();
          b->args.push_back(v);
          define(p.first, v);
        }
      sc.expect("{");
      ops_until(b.get(), "}");
      sc.expect("}");
      scopes.pop_back();
      op->regions.push_back(std::move(b));
      finish(op, results, rts);
      return;
    }
    if (sh == "while") {
      // stablehlo.while(%iterArg = %x, ...) : types [attributes {..}] cond { } do { }
      sc.expect("(");
      std::vector<std::string> names;
      if (!sc.accept(")")) {
        do {
          names.push_back(sc.ssa());
          sc.expect("=");
          op->operands.push_back(lookup(sc.ssa()));
        } while (sc.accept(","));
        sc.expect(")");
      }
      std::vector<TensorType> types;
      if (sc.accept(":")) { do { types.push_back(read_type(sc)); } while (sc.accept(",")); }
      if (sc.accept("attributes")) { sc.expect("{"); read_attr_dict(sc, "}", op->attrs); }
      for (const char* kw : {"cond", "do"}) {
        sc.expect(kw);
        sc.expect("{");
        auto b = std::make_unique<Block>();
        b->parent_op = op;
        scopes.emplace_back();
        for (size_t k = 0; k < names.size(); k++) {
          Value* v = m->new_value(types[k], names[k]);
          v->owner = b.get();
          v->arg_index = (int)k;
          b->args.push_back(v);
          define(names[k], v);
        }
        ops_until(b.get(), "}");
        sc.expect("}");
        scopes.pop_back();
        op->regions.push_back(std::move(b));
      }
      finish(op, results, types);
      return;
    }
    if (name == "call" || name == "func.call") {
      op->name = "func.call";
      sc.expect("@");
      op->attrs["callee"] = "@" + sc.ident();
      sc.expect("(");
      operand_list(op, ")");
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    auto functional_type = [&]() {
      sc.expect(":");
      read_type_list(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
    };
    auto keyword_dims = [&](const char* kw) {      // ", kw = [..]" -> array<i64: ..>
      sc.expect(",");
      sc.expect(kw);
      sc.expect("=");
      return dims_attr();
    };
    if (sh == "pad") {
      // stablehlo.pad %x, %value, low = [..], high = [..], interior = [..] : (types) -> type
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      op->operands.push_back(lookup(sc.ssa()));
      op->attrs["edge_padding_low"] = keyword_dims("low");
      op->attrs["edge_padding_high"] = keyword_dims("high");
      op->attrs["interior_padding"] = keyword_dims("interior");
      functional_type();
      return;
    }
    if (sh == "reverse") {
      // stablehlo.reverse %x, dims = [..] : type
      op->operands.push_back(lookup(sc.ssa()));
      op->attrs["dimensions"] = keyword_dims("dims");
      sc.expect(":");
      finish(op, results, {read_type(sc)});
      return;
    }
    if (sh == "reduce_precision") {
      // stablehlo.reduce_precision %x, format = e5m10 : type
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      sc.expect("format");
      sc.expect("=");
      const std::string f = sc.ident();
      const size_t mpos = f.find('m');
      if (f.size() < 4 || f[0] != 'e' || mpos == std::string::npos) sc.fail("reduce_precision: expected a format like e5m10");
      op->attrs["exponent_bits"] = f.substr(1, mpos - 1) + " : i32";
      op->attrs["mantissa_bits"] = f.substr(mpos + 1) + " : i32";
      sc.expect(":");
      finish(op, results, {read_type(sc)});
      return;
    }
    if (sh == "cholesky") {
      // stablehlo.cholesky %a[, lower = true] : type
      op->operands.push_back(lookup(sc.ssa()));
      if (sc.accept(",")) {
        sc.expect("lower");
        sc.expect("=");
        op->attrs["lower"] = sc.ident();
      }
      sc.expect(":");
      finish(op, results, {read_type(sc)});
      return;
    }
    if (sh == "rng_bit_generator") {
      // stablehlo.rng_bit_generator %state, algorithm = DEFAULT : (type) -> (type, type)
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      sc.expect("algorithm");
      sc.expect("=");
      op->attrs["rng_algorithm"] = "#stablehlo<rng_algorithm " + sc.ident() + ">";
      functional_type();
      return;
    }
    if (sh == "custom_call") {
      // stablehlo.custom_call @target(%a, %b) {attributes} : (types) -> types
      sc.expect("@");
      sc.ws();
      const std::string target = (sc.i < sc.n && sc.s[sc.i] == '"') ? sc.string_lit() : sc.ident();
      op->attrs["call_target_name"] = "\"" + target + "\"";
      sc.expect("(");
      operand_list(op, ")");
      if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
      functional_type();
      return;
    }
    if (sh == "after_all" || sh == "create_token" || sh == "partition_id" || sh == "replica_id") {
      // stablehlo.after_all %t0, %t1 : !stablehlo.token;  stablehlo.partition_id : tensor<ui32>
      while (sc.peek("%")) { op->operands.push_back(lookup(sc.ssa())); sc.accept(","); }
      sc.expect(":");
      finish(op, results, {read_type(sc)});
      return;
    }
    if (sh == "convolution") {
      // stablehlo.convolution(%lhs, %rhs) dim_numbers = [b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f],
      //   window = {stride = [..], pad = [[..], ..], lhs_dilate = [..], rhs_dilate = [..], reverse = [..]} {attributes} : (types) -> type
      sc.expect("(");
      operand_list(op, ")");
      sc.expect("dim_numbers");
      sc.expect("=");
      std::string dn;
      for (int part = 0; part < 3; part++) {
        sc.expect("[");
        dn += "[" + sc.balanced("]") + "]";
        sc.expect("]");
        if (part == 0) { sc.expect("x"); dn += "x"; }
        if (part == 1) { sc.expect("->"); dn += "->"; }
      }
      op->attrs["dimension_numbers"] = "#stablehlo.conv<" + dn + ">";
      sc.expect(",");
      sc.expect("window");
      sc.expect("=");
      sc.expect("{");
      if (!sc.accept("}")) {
        do {
          const std::string key = sc.ident();
          sc.expect("=");
          sc.expect("[");
          const std::string body = sc.balanced("]");
          sc.expect("]");
          if (key == "stride") op->attrs["window_strides"] = "array<i64: " + body + ">";
          else if (key == "lhs_dilate") op->attrs["lhs_dilation"] = "array<i64: " + body + ">";
          else if (key == "rhs_dilate") op->attrs["rhs_dilation"] = "array<i64: " + body + ">";
          else if (key == "reverse") op->attrs["window_reversal"] = "array<i1: " + body + ">";
          else if (key == "pad") {
            size_t pairs = 0;
            for (char ch : body) pairs += ch == '[';
            op->attrs["padding"] = "dense<[" + body + "]> : tensor<" + std::to_string(pairs) + "x2xi64>";
          } else sc.fail("convolution: unknown window entry '" + key + "'");
        } while (sc.accept(","));
        sc.expect("}");
      }
      if (sc.accept("{")) read_attr_dict(sc, "}", op->attrs);
      functional_type();
      return;
    }
    if (name == "chlo.top_k") {
      // chlo.top_k(%x, k = 3) : type -> (type, type)
      sc.expect("(");
      op->operands.push_back(lookup(sc.ssa()));
      sc.expect(",");
      sc.expect("k");
      sc.expect("=");
      op->attrs["k"] = std::to_string(sc.integer()) + " : i64";
      sc.expect(")");
      sc.expect(":");
      read_type(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    if (name.rfind("chlo.", 0) == 0 && sc.peek("%")) {
      // chlo.erf %x : type -> type (the unary functions; chlo's broadcasting binary operations are not accepted)
      op->operands.push_back(lookup(sc.ssa()));
      if (sc.peek(",")) sc.fail("custom assembly of '" + name + "' with several operands is not supported");
      sc.expect(":");
      read_type(sc);
      sc.expect("->");
      finish(op, results, read_type_list(sc));
      return;
    }
    sc.fail("custom assembly of '" + name + "' is not supported; print the module in generic form");
  }
};

}  // namespace

std::unique_ptr<Module> parse_module(const char* text, size_t size) {
  auto m = std::make_unique<Module>();
  ModuleParser p(text, size, m.get());
  p.parse();
  return m;
}

TensorType parse_type(const std::string& text) {
  Scanner sc(text.c_str(), text.size());
  return read_type(sc);
}

// ---------------------------------------------------------------------------
// attribute decoding
// ---------------------------------------------------------------------------
static std::string trim(const std::string& s) {
  size_t a = 0, b = s.size();
  while (a < b && isspace((unsigned char)s[a])) a++;
  while (b > a && isspace((unsigned char)s[b - 1])) b--;
  return s.substr(a, b - a);
}

int64_t attr_int(const std::string& raw) {
  std::string t = trim(raw);
  auto c = t.find(':');
  if (c != std::string::npos) t = trim(t.substr(0, c));
  if (t == "true") return 1;
  if (t == "false") return 0;
  return strtoll(t.c_str(), nullptr, 10);
}

bool attr_bool(const std::string& raw) {
  std::string t = trim(raw);
  auto c = t.find(':');
  if (c != std::string::npos) t = trim(t.substr(0, c));
  return t == "true" || t == "unit" || t == "1";
}

std::string attr_str(const std::string& raw) {
  std::string t = trim(raw);
  if (t.size() >= 2 && t[0] == '"') return t.substr(1, t.size() - 2);
  return t;
}

std::string attr_enum(const std::string& raw) {
  std::string t = trim(raw);
  while (!t.empty() && t.back() == '>') t.pop_back();
  auto p = t.find_last_of(" <");
  return p == std::string::npos ? t : t.substr(p + 1);
}

static std::vector<int64_t> ints_in(const std::string& s) {
  std::vector<int64_t> out;
  size_t i = 0;
  while (i < s.size()) {
    if (isdigit((unsigned char)s[i]) || ((s[i] == '-' || s[i] == '+') && i + 1 < s.size() && isdigit((unsigned char)s[i + 1]))) {
      size_t j = i + 1;
      while (j < s.size() && isdigit((unsigned char)s[j])) j++;
      out.push_back(strtoll(s.substr(i, j - i).c_str(), nullptr, 10));
      i = j;
    } else i++;
  }
  return out;
}

std::vector<int64_t> attr_i64s(const std::string& raw) {
  std::string t = trim(raw);
  if (t.rfind("array<", 0) == 0) {
    auto c = t.find(':');
    if (c == std::string::npos) return {};
    return ints_in(t.substr(c + 1));
  }
  if (t.rfind("dense<", 0) == 0) {
    DenseValue d = attr_dense(t);
    std::vector<int64_t> out;
    size_t n = (size_t)d.type.numel();
    for (size_t k = 0; k < n; k++) {
      const uint8_t* p = d.data.data() + k * dt_size(d.type.dt);
      switch (d.type.dt) {
        case DT::I64: case DT::U64: { int64_t v; memcpy(&v, p, 8); out.push_back(v); break; }
        case DT::I32: { int32_t v; memcpy(&v, p, 4); out.push_back(v); break; }
        case DT::U32: { uint32_t v; memcpy(&v, p, 4); out.push_back(v); break; }
        case DT::PRED: case DT::U8: out.push_back(*p); break;
        case DT::I8: out.push_back((int8_t)*p); break;
        default: throw CompileError("integer attribute of unsupported type " + d.type.str());
      }
    }
    return out;
  }
  if (!t.empty() && t[0] == '[') {
    // '[1, 2]' or '[1 : i64, 2 : i64]'
    std::vector<int64_t> out;
    std::string body = t.substr(1, t.size() - 2);
    std::stringstream ss(body);
    std::string item;
    while (std::getline(ss, item, ',')) {
      item = trim(item);
      if (!item.empty()) out.push_back(attr_int(item));
    }
    return out;
  }
  throw CompileError("cannot decode integer list attribute: " + t);
}

std::map<std::string, std::vector<int64_t>> attr_struct(const std::string& raw) {
  std::map<std::string, std::vector<int64_t>> out;
  auto lt = raw.find('<'), gt = raw.rfind('>');
  if (lt == std::string::npos || gt == std::string::npos) return out;
  std::string s = raw.substr(lt + 1, gt - lt - 1);
  size_t i = 0;
  while (i < s.size()) {
    while (i < s.size() && !(isalpha((unsigned char)s[i]) || s[i] == '_')) i++;
    size_t j = i;
    while (j < s.size() && (isalnum((unsigned char)s[j]) || s[j] == '_')) j++;
    if (j == i) break;
    std::string key = s.substr(i, j - i);
    i = j;
    while (i < s.size() && isspace((unsigned char)s[i])) i++;
    if (i >= s.size() || s[i] != '=') continue;
    i++;
    while (i < s.size() && isspace((unsigned char)s[i])) i++;
    if (i < s.size() && s[i] == '[') {
      size_t e = s.find(']', i);
      out[key] = ints_in(s.substr(i, e - i));
      i = e + 1;
    } else {
      size_t e = i;
      while (e < s.size() && s[e] != ',') e++;
      out[key] = ints_in(s.substr(i, e - i));
      i = e;
    }
  }
  return out;
}

static void store_scalar(DT dt, double fv, int64_t iv, uint64_t uv, bool is_float_tok, uint8_t* p) {
  switch (dt) {
    case DT::F32: { float f = is_float_tok ? (float)fv : (float)iv; memcpy(p, &f, 4); break; }
    case DT::F64: { double f = is_float_tok ? fv : (double)iv; memcpy(p, &f, 8); break; }
    case DT::BF16: { uint16_t h = f32_to_bf16(is_float_tok ? (float)fv : (float)iv); memcpy(p, &h, 2); break; }
    case DT::F16: { uint16_t h = f32_to_f16(is_float_tok ? (float)fv : (float)iv); memcpy(p, &h, 2); break; }
    case DT::PRED: *p = (uint8_t)(iv != 0); break;
    case DT::I8: case DT::U8: { int8_t v = (int8_t)iv; memcpy(p, &v, 1); break; }
    case DT::I16: case DT::U16: { int16_t v = (int16_t)iv; memcpy(p, &v, 2); break; }
    case DT::I32: case DT::U32: { int32_t v = (int32_t)(is_float_tok ? (int64_t)fv : iv); memcpy(p, &v, 4); break; }
    case DT::I64: { memcpy(p, &iv, 8); break; }
    case DT::U64: { memcpy(p, &uv, 8); break; }
    default: throw CompileError("dense constant of unsupported element type");
  }
}

DenseValue attr_dense(const std::string& raw_in) {
  std::string raw = trim(raw_in);
  if (raw.rfind("dense<", 0) != 0) throw CompileError("expected dense<...> attribute, got: " + raw.substr(0, 40));
  Scanner sc(raw.c_str(), raw.size());
  sc.i = 6;
  std::string body = sc.balanced(">");
  sc.expect(">");
  sc.expect(":");
  DenseValue d;
  d.type = read_type(sc);
  size_t es = dt_size(d.type.dt);
  size_t n = (size_t)d.type.numel();
  d.data.assign(n * es, 0);
  if (body.size() >= 3 && body[0] == '"' && body[1] == '0' && body[2] == 'x') {
    std::string hex = body.substr(3, body.size() - 4);
    std::vector<uint8_t> bytes(hex.size() / 2);
    auto nib = [](char c) -> int { return c <= '9' ? c - '0' : (c | 0x20) - 'a' + 10; };
    for (size_t k = 0; k < bytes.size(); k++) bytes[k] = (uint8_t)(nib(hex[2 * k]) * 16 + nib(hex[2 * k + 1]));
    if (d.type.dt == DT::PRED && bytes.size() != n && bytes.size() * 8 >= n && bytes.size() != 1) {
      for (size_t k = 0; k < n; k++) d.data[k] = (bytes[k / 8] >> (k % 8)) & 1;     // bit-packed legacy form
    } else if (bytes.size() == n * es) {
      d.data = bytes;
      if (d.type.dt == DT::PRED) for (auto& b : d.data) b = b != 0;
    } else if (bytes.size() == es) {
      for (size_t k = 0; k < n; k++) memcpy(d.data.data() + k * es, bytes.data(), es);
      if (d.type.dt == DT::PRED) for (auto& b : d.data) b = b != 0;
    } else throw CompileError("dense hex blob size mismatch for " + d.type.str());
  } else {
    // token scan: numbers, true/false, hex bit patterns
    size_t count = 0, i = 0;
    std::vector<uint8_t> one(es ? es : 1);
    auto put = [&](double fv, int64_t iv, uint64_t uv, bool isf) {
      if (count < n) store_scalar(d.type.dt, fv, iv, uv, isf, d.data.data() + count * es);
      else if (n == 0) {}
      count++;
    };
    while (i < body.size()) {
      char c = body[i];
      if (body.compare(i, 4, "true") == 0) { put(1, 1, 1, false); i += 4; }
      else if (body.compare(i, 5, "false") == 0) { put(0, 0, 0, false); i += 5; }
      else if (isdigit((unsigned char)c) || c == '-' || c == '+' || c == '.' ||
               body.compare(i, 3, "inf") == 0 || body.compare(i, 3, "nan") == 0) {
        size_t j = i;
        if (body[j] == '-' || body[j] == '+') j++;
        if (body.compare(j, 2, "0x") == 0) {
          size_t k = j + 2;
          while (k < body.size() && isxdigit((unsigned char)body[k])) k++;
          uint64_t bits = strtoull(body.substr(j + 2, k - j - 2).c_str(), nullptr, 16);
          if (dt_is_float(d.type.dt)) {           // bit pattern of the element type
            if (count < n) memcpy(d.data.data() + count * es, &bits, es);
            count++;
          } else put(0, (int64_t)bits, bits, false);
          i = k;
        } else {
          size_t k = j;
          bool isf = false;
          while (k < body.size() && (isalnum((unsigned char)body[k]) || body[k] == '.' ||
                                     ((body[k] == '-' || body[k] == '+') && (body[k - 1] == 'e' || body[k - 1] == 'E')))) {
            if (body[k] == '.' || body[k] == 'e' || body[k] == 'E' || body[k] == 'n' || body[k] == 'i') isf = true;
            k++;
          }
          std::string tok = body.substr(i, k - i);
          if (isf) put(strtod(tok.c_str(), nullptr), 0, 0, true);
          else {
            bool neg = tok[0] == '-';
            uint64_t uv = strtoull(tok.c_str() + (neg || tok[0] == '+' ? 1 : 0), nullptr, 10);
            int64_t iv = neg ? -(int64_t)uv : (int64_t)uv;
            put((double)iv, iv, neg ? (uint64_t)iv : uv, false);
          }
          i = k;
        }
      } else i++;
    }
    if (count == 1 && n != 1) {
      for (size_t k = 1; k < n; k++) memcpy(d.data.data() + k * es, d.data.data(), es);
    } else if (count != n && !(n == 0)) {
      throw CompileError("dense constant has " + std::to_string(count) + " elements, type needs " + std::to_string(n));
    }
  }
  d.splat = true;
  for (size_t k = 1; k < n && d.splat; k++)
    if (memcmp(d.data.data(), d.data.data() + k * es, es) != 0) d.splat = false;
  return d;
}

}  // namespace b200
