// CUDA source generation for fused kernels (see codegen.h).
#include "codegen.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace b200 {

const char* c_type(DT d) {
  switch (d) {
    case DT::PRED: return "bool";
    case DT::I8: return "i8";
    case DT::I16: return "i16";
    case DT::I32: return "i32";
    case DT::I64: return "i64";
    case DT::U8: return "u8";
    case DT::U16: return "u16";
    case DT::U32: return "u32";
    case DT::U64: return "u64";
    case DT::F16: case DT::BF16: case DT::F32: return "float";
    case DT::F64: return "double";
    default: throw CompileError("no register type for element type");
  }
}

const char* s_type(DT d) {
  switch (d) {
    case DT::PRED: return "u8";
    case DT::F16: case DT::BF16: return "u16";
    default: return c_type(d);
  }
}

static std::string float_lit(float f) {
  if (std::isnan(f) || std::isinf(f)) {
    uint32_t u;
    memcpy(&u, &f, 4);
    char buf[48];
    snprintf(buf, sizeof buf, "__uint_as_float(0x%08Xu)", u);
    return buf;
  }
  char buf[64];
  snprintf(buf, sizeof buf, "%af", (double)f);
  return buf;
}

std::string literal(DT d, const uint8_t* p) {
  char buf[96];
  switch (d) {
    case DT::PRED: return *p ? "true" : "false";
    case DT::I8: { int8_t v; memcpy(&v, p, 1); return "(i8)" + std::to_string((int)v); }
    case DT::U8: return "(u8)" + std::to_string((unsigned)*p);
    case DT::I16: { int16_t v; memcpy(&v, p, 2); return "(i16)" + std::to_string((int)v); }
    case DT::U16: { uint16_t v; memcpy(&v, p, 2); return "(u16)" + std::to_string((unsigned)v); }
    case DT::I32: { int32_t v; memcpy(&v, p, 4); snprintf(buf, sizeof buf, "(i32)0x%08Xu", (uint32_t)v); return buf; }
    case DT::U32: { uint32_t v; memcpy(&v, p, 4); snprintf(buf, sizeof buf, "0x%08Xu", v); return buf; }
    case DT::I64: { uint64_t v; memcpy(&v, p, 8); snprintf(buf, sizeof buf, "(i64)0x%016llXull", (unsigned long long)v); return buf; }
    case DT::U64: { uint64_t v; memcpy(&v, p, 8); snprintf(buf, sizeof buf, "0x%016llXull", (unsigned long long)v); return buf; }
    case DT::F32: { float f; memcpy(&f, p, 4); return float_lit(f); }
    case DT::BF16: { uint16_t h; memcpy(&h, p, 2); return float_lit(bf16_to_f32(h)); }
    case DT::F16: { uint16_t h; memcpy(&h, p, 2); return float_lit(f16_to_f32(h)); }
    case DT::F64: {
      double f; memcpy(&f, p, 8);
      if (std::isnan(f) || std::isinf(f)) {
        uint64_t u; memcpy(&u, &f, 8);
        snprintf(buf, sizeof buf, "__longlong_as_double(0x%016llXll)", (unsigned long long)u);
      } else snprintf(buf, sizeof buf, "%a", f);
      return buf;
    }
    default: throw CompileError("literal of unsupported type");
  }
}

static const std::map<std::string, const char*>& binary_fn() {
  static const std::map<std::string, const char*> m = {
      {"add", "op_add"}, {"subtract", "op_sub"}, {"multiply", "op_mul"}, {"divide", "op_div"},
      {"remainder", "op_rem"}, {"maximum", "op_max"}, {"minimum", "op_min"}, {"power", "op_pow"},
      {"atan2", "op_atan2"}, {"and", "op_and"}, {"or", "op_or"}, {"xor", "op_xor"},
      {"shift_left", "op_shl"}, {"shift_right_logical", "op_shrl"}, {"shift_right_arithmetic", "op_shra"}};
  return m;
}
static const std::map<std::string, const char*>& unary_fn() {
  static const std::map<std::string, const char*> m = {
      {"exponential", "op_exp"}, {"log", "op_log"}, {"sqrt", "op_sqrt"}, {"rsqrt", "op_rsqrt"},
      {"negate", "op_neg"}, {"abs", "op_abs"}, {"floor", "op_floor"}, {"ceil", "op_ceil"},
      {"sine", "op_sin"}, {"cosine", "op_cos"}, {"tan", "op_tan"}, {"tanh", "op_tanh"},
      {"logistic", "op_logistic"}, {"sign", "op_sign"}, {"log_plus_one", "op_log1p"},
      {"exponential_minus_one", "op_expm1"}, {"cbrt", "op_cbrt"}, {"not", "op_not"}, {"popcnt", "op_popcnt"},
      {"count_leading_zeros", "op_clz"}, {"round_nearest_even", "op_rne"}, {"round_nearest_afz", "op_rafz"},
      {"is_finite", "op_isfinite"}, {"erf", "op_erf"}, {"sinh", "op_sinh"}, {"cosh", "op_cosh"}, {"asin", "op_asin"},
      {"acos", "op_acos"}, {"atan", "op_atan"}, {"asinh", "op_asinh"}, {"acosh", "op_acosh"}, {"atanh", "op_atanh"},
      {"erf_inv", "op_erfinv"}};
  return m;
}

bool is_elementwise_op(const std::string& s) {
  return binary_fn().count(s) || unary_fn().count(s) || s == "compare" || s == "select" || s == "clamp" ||
         s == "convert" || s == "bitcast_convert" || s == "reduce_precision";
}

void Emitter::line(const std::string& s) { os_ << std::string(indent_, ' ') << s << "\n"; }
std::string Emitter::fresh(const char* p) { return name_prefix + p + std::to_string(nvar_++); }

std::string Emitter::input_name(Value* v) {
  auto it = in_index_.find(v);
  if (it == in_index_.end()) {
    in_index_[v] = (int)inputs.size();
    inputs.push_back(v);
    return "in" + std::to_string(inputs.size() - 1);
  }
  return "in" + std::to_string(it->second);
}

void Emitter::ensure_idx(Ctx& c) {
  if (c.idx.size() == c.shape.size()) return;
  c.idx.assign(c.shape.size(), "0");
  int64_t stride = 1;
  std::vector<int64_t> strides(c.shape.size());
  for (int d = (int)c.shape.size() - 1; d >= 0; d--) { strides[d] = stride; stride *= c.shape[d]; }
  for (size_t d = 0; d < c.shape.size(); d++) {
    if (c.shape[d] == 1) continue;
    std::string v = fresh("x");
    std::string e = c.lin;
    if (strides[d] != 1) e = "(" + e + " / " + std::to_string(strides[d]) + ")";
    if (d != 0) {
      bool leading_all_one = true;
      for (size_t q = 0; q < d; q++) leading_all_one &= c.shape[q] == 1;
      if (!leading_all_one) e = "(" + e + " % " + std::to_string(c.shape[d]) + ")";
    }
    line("const " + idx_t + " " + v + " = " + e + ";");
    c.idx[d] = v;
  }
}

std::string Emitter::lin_of(Ctx& c) {
  if (!c.lin.empty()) return c.lin;
  if (c.shape.empty()) { c.lin = "0"; return c.lin; }
  std::string e;
  int64_t stride = 1;
  std::vector<std::string> terms;
  for (int d = (int)c.shape.size() - 1; d >= 0; d--) {
    if (c.shape[d] != 1 && c.idx[d] != "0")
      terms.push_back(stride == 1 ? c.idx[d] : "(" + idx_t + ")" + c.idx[d] + " * " + std::to_string(stride));
    stride *= c.shape[d];
  }
  if (terms.empty()) { c.lin = "0"; return c.lin; }
  for (size_t k = 0; k < terms.size(); k++) e += (k ? " + " : "") + terms[k];
  std::string v = fresh("l");
  line("const " + idx_t + " " + v + " = " + e + ";");
  c.lin = v;
  return v;
}

std::string Emitter::key(Value* v, Ctx& c) {
  std::string k = std::to_string(v->id) + "@";
  if (!c.lin.empty()) return k + "L" + c.lin;
  for (auto& s : c.idx) k += s + ",";
  return k;
}

std::string Emitter::load(Value* v, Ctx& c) {
  std::string p = input_name(v);
  std::string at = lin_of(c);
  DT d = v->type.dt;
  std::string var = fresh("v");
  std::string e = p + "[" + at + "]";
  if (d == DT::BF16) e = "bf16_to_f(" + e + ")";
  else if (d == DT::F16) e = "f16_to_f(" + e + ")";
  else if (d == DT::PRED) e = "(" + e + " != 0)";
  line(std::string("const ") + c_type(d) + " " + var + " = " + e + ";");
  return var;
}

std::string Emitter::elementwise(Op* op, const std::vector<std::string>& a) {
  std::string sh = op->short_name();
  DT rt = op->results[0]->type.dt;
  DT it = op->operands.empty() ? rt : op->operands[0]->type.dt;
  std::string e;
  auto bf = binary_fn().find(sh);
  auto uf = unary_fn().find(sh);
  if (bf != binary_fn().end()) e = std::string(bf->second) + "(" + a[0] + ", " + a[1] + ")";
  else if (uf != unary_fn().end()) e = std::string(uf->second) + "(" + a[0] + ")";
  else if (sh == "compare") {
    std::string dir = attr_enum(op->attr("comparison_direction"));
    bool total = op->has("compare_type") && attr_enum(op->attr("compare_type")) == "TOTALORDER" && dt_is_float(it);
    if (total) e = "cmp_" + dir + "(tkey(" + a[0] + "), tkey(" + a[1] + "))";
    else e = "cmp_" + dir + "(" + a[0] + ", " + a[1] + ")";
  } else if (sh == "select") e = "(" + a[0] + " ? " + a[1] + " : " + a[2] + ")";
  else if (sh == "clamp") e = "op_min(op_max(" + a[1] + ", " + a[0] + "), " + a[2] + ")";
  else if (sh == "convert") e = std::string("cvt<") + c_type(rt) + ", " + c_type(it) + ">(" + a[0] + ")";
  else if (sh == "bitcast_convert") {
    if (dt_size(rt) != dt_size(it)) throw CompileError("bitcast_convert between different widths is not supported");
    std::string src = a[0];
    const char* from = c_type(it);
    if (it == DT::BF16) { src = "f_to_bf16(" + src + ")"; from = "u16"; }
    if (it == DT::F16) { src = "f_to_f16(" + src + ")"; from = "u16"; }
    if (rt == DT::BF16) e = "bf16_to_f(bitcast<u16, " + std::string(from) + ">(" + src + "))";
    else if (rt == DT::F16) e = "f16_to_f(bitcast<u16, " + std::string(from) + ">(" + src + "))";
    else if (rt == DT::PRED || it == DT::PRED) throw CompileError("bitcast_convert of i1");
    else e = std::string("bitcast<") + c_type(rt) + ", " + from + ">(" + src + ")";
    return e;
  } else if (sh == "reduce_precision") {
    e = "reduce_prec(" + a[0] + ", " + std::to_string(attr_int(op->attr("exponent_bits"))) + ", " +
        std::to_string(attr_int(op->attr("mantissa_bits"))) + ")";
  } else throw CompileError("no code generation rule for " + op->name);
  if (round_small_floats) {
    if (rt == DT::BF16) e = "rbf16(" + e + ")";
    else if (rt == DT::F16) e = "rf16(" + e + ")";
  }
  return e;
}

std::vector<std::string> Emitter::emit_scalar_region(Block* b, const std::vector<std::string>& args) {
  std::map<Value*, std::string> env;
  for (size_t k = 0; k < b->args.size(); k++) env[b->args[k]] = args[k];
  for (auto& op : b->ops) {
    std::string sh = op->short_name();
    if (sh == "return") {
      std::vector<std::string> out;
      for (auto* v : op->operands) {
        auto it = env.find(v);
        if (it == env.end()) throw CompileError("region result defined outside the region is not supported");
        out.push_back(it->second);
      }
      return out;
    }
    std::string e;
    DT rt = op->results[0]->type.dt;
    if (sh == "constant") {
      DenseValue d = attr_dense(op->attr("value"));
      e = literal(d.type.dt, d.data.data());
    } else if (is_elementwise_op(sh)) {
      std::vector<std::string> a;
      for (auto* v : op->operands) {
        auto it = env.find(v);
        if (it == env.end()) throw CompileError("region of " + b->parent_op->name + " uses a value defined outside it");
        a.push_back(it->second);
      }
      e = elementwise(op.get(), a);
    } else throw CompileError("operation " + op->name + " inside a combiner region is not supported");
    std::string var = fresh("c");
    line(std::string("const ") + c_type(rt) + " " + var + " = " + e + ";");
    env[op->results[0]] = var;
  }
  throw CompileError("region without return");
}

std::string Emitter::emit(Value* v, Ctx c) {
  auto bit = bound.find(v);
  if (bit != bound.end()) return bit->second;
  Op* d = v->def;
  if (!d || !is_internal(d)) {
    std::string at = lin_of(c);
    std::string k = std::to_string(v->id) + "@L" + at;
    for (auto it = memo_.rbegin(); it != memo_.rend(); ++it) {
      auto f = it->find(k);
      if (f != it->end()) return f->second;
    }
    std::string var = load(v, c);
    memo_.back()[k] = var;
    return var;
  }
  std::string k = key(v, c);
  for (auto it = memo_.rbegin(); it != memo_.rend(); ++it) {
    auto f = it->find(k);
    if (f != it->end()) return f->second;
  }
  std::string sh = d->short_name();
  DT rt = v->type.dt;
  std::string ct = c_type(rt);
  std::string var;
  auto same_ctx = [&](Value* o) -> Ctx {
    if (o->type.dims == c.shape) return c;
    if (o->type.rank() == 0) { Ctx s; s.lin = "0"; return s; }
    throw CompileError(d->name + ": operand shape differs from result shape");
  };
  if (is_elementwise_op(sh)) {
    std::vector<std::string> a;
    for (auto* o : d->operands) a.push_back(emit(o, same_ctx(o)));
    var = fresh("v");
    line("const " + ct + " " + var + " = " + elementwise(d, a) + ";");
  } else if (sh == "constant") {
    DenseValue dv = attr_dense(d->attr("value"));
    if (!dv.splat) throw CompileError("internal: non-splat constant inside a fusion");
    var = literal(dv.type.dt, dv.data.data());
    return var;
  } else if (sh == "iota") {
    ensure_idx(c);
    int dim = (int)attr_int(d->attr("iota_dimension"));
    var = fresh("v");
    line("const " + ct + " " + var + " = (" + ct + ")" + c.idx[dim] + ";");
  } else if (sh == "broadcast_in_dim") {
    ensure_idx(c);
    auto dims = attr_i64s(d->attr("broadcast_dimensions"));
    Value* o = d->operands[0];
    Ctx oc;
    oc.shape = o->type.dims;
    oc.idx.resize(dims.size());
    for (size_t i = 0; i < dims.size(); i++)
      oc.idx[i] = (o->type.dims[i] == 1) ? "0" : c.idx[dims[i]];
    if (oc.shape.empty()) oc.lin = "0";
    return emit(o, oc);
  } else if (sh == "reshape") {
    Value* o = d->operands[0];
    Ctx oc;
    oc.shape = o->type.dims;
    oc.lin = lin_of(c);
    return emit(o, oc);
  } else if (sh == "transpose") {
    ensure_idx(c);
    auto perm = attr_i64s(d->attr("permutation"));
    Value* o = d->operands[0];
    Ctx oc;
    oc.shape = o->type.dims;
    oc.idx.resize(perm.size());
    for (size_t i = 0; i < perm.size(); i++) oc.idx[perm[i]] = c.idx[i];
    return emit(o, oc);
  } else if (sh == "reverse") {
    ensure_idx(c);
    auto dims = attr_i64s(d->attr("dimensions"));
    Ctx oc = c;
    oc.lin.clear();
    for (auto dd : dims) {
      if (c.shape[dd] == 1) continue;
      std::string nv = fresh("x");
      line("const " + idx_t + " " + nv + " = " + std::to_string(c.shape[dd] - 1) + " - " + c.idx[dd] + ";");
      oc.idx[dd] = nv;
    }
    return emit(d->operands[0], oc);
  } else if (sh == "slice") {
    ensure_idx(c);
    auto st = attr_i64s(d->attr("start_indices"));
    auto sd = attr_i64s(d->attr("strides"));
    Value* o = d->operands[0];
    Ctx oc;
    oc.shape = o->type.dims;
    oc.idx = c.idx;
    for (size_t i = 0; i < st.size(); i++) {
      if (st[i] == 0 && sd[i] == 1) continue;
      if (c.shape[i] == 1) { oc.idx[i] = std::to_string(st[i]); continue; }
      std::string nv = fresh("x");
      line("const " + idx_t + " " + nv + " = " + c.idx[i] + " * " + std::to_string(sd[i]) + " + " + std::to_string(st[i]) + ";");
      oc.idx[i] = nv;
    }
    return emit(o, oc);
  } else if (sh == "pad") {
    ensure_idx(c);
    auto lo = attr_i64s(d->attr("edge_padding_low"));
    auto in = attr_i64s(d->attr("interior_padding"));
    Value* o = d->operands[0];
    Ctx sc;
    sc.lin = "0";
    std::string pv = emit(d->operands[1], sc);
    Ctx oc;
    oc.shape = o->type.dims;
    oc.idx = c.idx;
    std::string ok = fresh("ok");
    line("bool " + ok + " = true;");
    for (size_t i = 0; i < lo.size(); i++) {
      int64_t step = in[i] + 1;
      bool trivial = lo[i] == 0 && step == 1 && o->type.dims[i] == c.shape[i];
      if (trivial) continue;
      std::string t = fresh("x");
      line("const " + idx_t + " " + t + " = " + c.idx[i] + " - (" + std::to_string(lo[i]) + ");");
      std::string q = t;
      if (step != 1) {
        q = fresh("x");
        line("const " + idx_t + " " + q + " = " + t + " / " + std::to_string(step) + ";");
        line(ok + " = " + ok + " && (" + t + " % " + std::to_string(step) + " == 0);");
      }
      line(ok + " = " + ok + " && " + t + " >= 0 && " + q + " < " + std::to_string(o->type.dims[i]) + ";");
      oc.idx[i] = q;
    }
    var = fresh("v");
    line(ct + " " + var + " = " + pv + ";");
    line("if (" + ok + ") {");
    push_scope();
    std::string x = emit(o, oc);
    line(var + " = " + x + ";");
    pop_scope();
    line("}");
  } else if (sh == "concatenate") {
    ensure_idx(c);
    int dim = (int)attr_int(d->attr("dimension"));
    var = fresh("v");
    line(ct + " " + var + ";");
    int64_t off = 0;
    for (size_t k = 0; k < d->operands.size(); k++) {
      Value* o = d->operands[k];
      int64_t sz = o->type.dims[dim];
      if (sz == 0) continue;
      bool last = true;
      for (size_t q = k + 1; q < d->operands.size(); q++) last &= d->operands[q]->type.dims[dim] == 0;
      std::string cond = last ? "" : "if (" + c.idx[dim] + " < " + std::to_string(off + sz) + ") ";
      line((off == 0 ? "" : "else ") + cond + "{");
      push_scope();
      Ctx oc;
      oc.shape = o->type.dims;
      oc.idx = c.idx;
      if (off != 0) {
        std::string nv = fresh("x");
        line("const " + idx_t + " " + nv + " = " + c.idx[dim] + " - " + std::to_string(off) + ";");
        oc.idx[dim] = nv;
      }
      std::string x = emit(o, oc);
      line(var + " = " + x + ";");
      pop_scope();
      line("}");
      off += sz;
    }
  } else if (sh == "dynamic_slice" || sh == "dynamic_update_slice") {
    ensure_idx(c);
    bool upd = sh == "dynamic_update_slice";
    Value* o = d->operands[0];
    size_t first = upd ? 2 : 1;
    const std::vector<int64_t>& win = upd ? d->operands[1]->type.dims : c.shape;
    std::vector<std::string> starts;
    Ctx sc;
    sc.lin = "0";
    for (size_t i = 0; i < o->type.dims.size(); i++) {
      std::string s = emit(d->operands[first + i], sc);
      std::string nv = fresh("s");
      // clamp into [0, dim - window] (src/pjrt_plugin/ops/slice.cc:80-107)
      line("const " + idx_t + " " + nv + " = (" + idx_t + ")min(max((i64)" + s + ", (i64)0), (i64)" +
           std::to_string(o->type.dims[i] - win[i]) + ");");
      starts.push_back(nv);
    }
    if (!upd) {
      Ctx oc;
      oc.shape = o->type.dims;
      oc.idx.resize(starts.size());
      for (size_t i = 0; i < starts.size(); i++) {
        std::string nv = fresh("x");
        line("const " + idx_t + " " + nv + " = " + c.idx[i] + " + " + starts[i] + ";");
        oc.idx[i] = nv;
      }
      return emit(o, oc);
    }
    Value* u = d->operands[1];
    std::string in = fresh("ok");
    line("bool " + in + " = true;");
    Ctx uc;
    uc.shape = u->type.dims;
    uc.idx.resize(starts.size());
    for (size_t i = 0; i < starts.size(); i++) {
      std::string nv = fresh("x");
      line("const " + idx_t + " " + nv + " = " + c.idx[i] + " - " + starts[i] + ";");
      line(in + " = " + in + " && " + nv + " >= 0 && " + nv + " < " + std::to_string(u->type.dims[i]) + ";");
      uc.idx[i] = nv;
    }
    var = fresh("v");
    line(ct + " " + var + ";");
    line("if (" + in + ") {");
    push_scope();
    line(var + " = " + emit(u, uc) + ";");
    pop_scope();
    line("} else {");
    push_scope();
    Ctx oc = c;
    line(var + " = " + emit(o, oc) + ";");
    pop_scope();
    line("}");
  } else if (sh == "gather") {
    // General gather: start indices clamped into [0, dim - slice_size]; the
    // operand must be external (src/pjrt_plugin/ops/gather_scatter.cc:200-294).
    ensure_idx(c);
    auto f = attr_struct(d->attr("dimension_numbers"));
    auto sizes = attr_i64s(d->attr("slice_sizes"));
    Value* operand = d->operands[0];
    Value* indices = d->operands[1];
    auto offset_dims = f["offset_dims"], collapsed = f["collapsed_slice_dims"], obatch = f["operand_batching_dims"],
         ibatch = f["start_indices_batching_dims"], smap = f["start_index_map"];
    int64_t ivd = f.count("index_vector_dim") ? f["index_vector_dim"][0] : indices->type.rank();
    int out_rank = (int)c.shape.size();
    std::vector<int> batch_out;     // output dims that index the batch of start_indices
    for (int q = 0; q < out_rank; q++)
      if (std::find(offset_dims.begin(), offset_dims.end(), q) == offset_dims.end()) batch_out.push_back(q);
    std::vector<int> idx_batch_dims;
    for (int q = 0; q < indices->type.rank(); q++)
      if (q != ivd) idx_batch_dims.push_back(q);
    std::vector<std::string> full(operand->type.rank(), "0");
    for (size_t kk = 0; kk < smap.size(); kk++) {
      Ctx ic;
      ic.shape = indices->type.dims;
      ic.idx.assign(indices->type.rank(), "0");
      for (size_t q = 0; q < idx_batch_dims.size(); q++) ic.idx[idx_batch_dims[q]] = c.idx[batch_out[q]];
      if (ivd < indices->type.rank()) ic.idx[ivd] = std::to_string(kk);
      std::string s = emit(indices, ic);
      int od = (int)smap[kk];
      std::string nv = fresh("g");
      line("const " + idx_t + " " + nv + " = (" + idx_t + ")min(max((i64)" + s + ", (i64)0), (i64)" +
           std::to_string(operand->type.dims[od] - sizes[od]) + ");");
      full[od] = nv;
    }
    for (size_t q = 0; q < obatch.size(); q++) {
      size_t pos = std::find(idx_batch_dims.begin(), idx_batch_dims.end(), (int)ibatch[q]) - idx_batch_dims.begin();
      full[obatch[q]] = c.idx[batch_out[pos]];
    }
    int w = 0;
    for (int od = 0; od < operand->type.rank(); od++) {
      if (std::find(collapsed.begin(), collapsed.end(), od) != collapsed.end()) continue;
      if (std::find(obatch.begin(), obatch.end(), od) != obatch.end()) continue;
      std::string o_idx = c.idx[offset_dims[w++]];
      if (full[od] == "0") full[od] = o_idx;
      else if (o_idx != "0") {
        std::string nv = fresh("g");
        line("const " + idx_t + " " + nv + " = " + full[od] + " + " + o_idx + ";");
        full[od] = nv;
      }
    }
    Ctx oc;
    oc.shape = operand->type.dims;
    oc.idx = full;
    return emit(operand, oc);
  } else {
    throw CompileError("internal: op " + d->name + " cannot be generated inside a fusion");
  }
  memo_.back()[k] = var;
  return var;
}

}  // namespace b200
