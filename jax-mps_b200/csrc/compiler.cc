// StableHLO module -> kernel plan.
//
// Pipeline (the reference's counterpart is finalizeModule + MpsFusionPass +
// the trace-and-replay executor: src/pjrt_plugin/stablehlo_parser.cc:80-285,
// src/pjrt_plugin/mlx_executable.cc:619-1008):
//   1. inline func.call / stablehlo.composite, drop pass-through ops
//      (optimization_barrier, Sharding custom calls), fold identity broadcasts;
//   2. reject unsupported operations with one error naming all of them;
//   3. group fusable operations (elementwise, index-rewriting, reductions with
//      their producers) into generated kernels;
//   4. order the units, give every materialised tensor a slot and lay the
//      temporaries out in an arena by liveness;
//   5. lower dot_general and convolution to the table-driven implicit-GEMM kernel.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <queue>
#include <regex>
#include <set>
#include <tuple>
#include <sstream>

#include "codegen.h"
#include "plan.h"

namespace b200 {

const char* codegen_prelude() {
  static const char* s =
#include "prelude.inc"
      ;
  return s;
}

namespace {

// ---------------------------------------------------------------------------
// dot_general on two 16-bit floating-point operands of one type: geometry for the native kernels (gemm16.cu)
// ---------------------------------------------------------------------------
// Each operand must be a strided matrix per batch group: its batch, free and contracting dimensions each collapse
// to one stride, and m or k (n or k) is contiguous. An operand whose row stride is not a multiple of 16 bytes
// (a vocabulary of 30522 columns) is copied once into rows padded to a multiple of eight elements, which TMA can
// address; what the padding holds never matters, the copy engine reads zeros outside the declared extent.
struct Dot16 {
  Gemm16Launch g;
  struct Repack { bool needed = false; long long rows = 0, cols = 0, src_ld = 0, dst_ld = 0; } ra, rb;
};

bool dot16_geometry(Op* op, Dot16& d) {
  if (op->operands.size() != 2 || op->results.size() != 1 || getenv("B200_NO_GEMM16")) return false;
  Value *lhs = op->operands[0], *rhs = op->operands[1], *out = op->results[0];
  const DT dt = lhs->type.dt;
  if (dt != rhs->type.dt || !(dt == DT::BF16 || dt == DT::F16)) return false;
  if (!(out->type.dt == dt || out->type.dt == DT::F32)) return false;
  if (!op->has("dot_dimension_numbers")) return false;
  auto f = attr_struct(op->attr("dot_dimension_numbers"));
  auto lbd = f["lhs_batching_dimensions"], rbd = f["rhs_batching_dimensions"];
  auto lcd = f["lhs_contracting_dimensions"], rcd = f["rhs_contracting_dimensions"];
  auto in = [](const std::vector<int64_t>& v, int64_t x) { return std::find(v.begin(), v.end(), x) != v.end(); };
  std::vector<int64_t> lfree, rfree;
  for (int k = 0; k < lhs->type.rank(); k++) if (!in(lbd, k) && !in(lcd, k)) lfree.push_back(k);
  for (int k = 0; k < rhs->type.rank(); k++) if (!in(rbd, k) && !in(rcd, k)) rfree.push_back(k);
  auto strides = [](const std::vector<int64_t>& dims) {
    std::vector<int64_t> s(dims.size());
    int64_t st = 1;
    for (int k = (int)dims.size() - 1; k >= 0; k--) { s[k] = st; st *= dims[k]; }
    return s;
  };
  // the row-major multi-index over `which` as extent and a single stride (false when it does not collapse)
  auto collapse = [](const std::vector<int64_t>& dims, const std::vector<int64_t>& s, const std::vector<int64_t>& which,
                     long long& extent, long long& stride) {
    extent = 1;
    stride = 0;
    bool have = false;
    for (int q = (int)which.size() - 1; q >= 0; q--) {
      const int64_t dsz = dims[which[q]];
      if (dsz == 1) continue;
      if (!have) { stride = s[which[q]]; have = true; }
      else if (s[which[q]] != stride * extent) return false;
      extent *= dsz;
    }
    return true;
  };
  auto sl = strides(lhs->type.dims), sr = strides(rhs->type.dims);
  long long G, G2, M, N, K, K2;
  Gemm16Launch& g = d.g;
  if (!collapse(lhs->type.dims, sl, lbd, G, g.a_gs) || !collapse(rhs->type.dims, sr, rbd, G2, g.b_gs) ||
      !collapse(lhs->type.dims, sl, lfree, M, g.a_ms) || !collapse(rhs->type.dims, sr, rfree, N, g.b_ns) ||
      !collapse(lhs->type.dims, sl, lcd, K, g.a_ks) || !collapse(rhs->type.dims, sr, rcd, K2, g.b_ks))
    return false;
  if (G != G2 || K != K2 || G <= 0 || M <= 0 || N <= 0 || K < 8) return false;
  if (G > 65535 || M >= (1LL << 31) || N >= (1LL << 31) || K >= (1LL << 31)) return false;
  // an index of extent 1 has no stride of its own: give it the one that makes the operand a plain matrix
  if (K == 1) return false;
  if (M == 1) g.a_ms = g.a_ks == 1 ? K : 1;
  if (N == 1) g.b_ns = g.b_ks == 1 ? K : 1;
  g.M = (int)M; g.N = (int)N; g.K = (int)K; g.G = (int)G;
  g.in_fmt = dt == DT::BF16 ? 1 : 0;
  g.c_kind = out->type.dt == DT::F32 ? 2 : g.in_fmt;
  if (!((g.a_ks == 1 || g.a_ms == 1) && (g.b_ks == 1 || g.b_ns == 1))) return false;
  if (M <= 8) {
    Gemm16Launch t = g;
    if (gemm16_plan(t, false) && t.path != 0) { g = t; return true; }
  }
  // tensor-core tiles: TMA needs 16-byte strides
  auto fix = [&](long long& ld, long long& gs, long long outer, long long inner, Dot16::Repack& r) {
    if (ld % 8 == 0 && (G == 1 || gs % 8 == 0)) return true;
    if (!(G == 1 || gs == outer * ld)) return false;        // groups must continue the rows
    r.needed = true;
    r.rows = G * outer;
    r.cols = inner;
    r.src_ld = ld;
    r.dst_ld = (inner + 7) / 8 * 8;
    ld = r.dst_ld;
    gs = outer * r.dst_ld;
    return true;
  };
  if (g.a_ks == 1) { if (!fix(g.a_ms, g.a_gs, M, K, d.ra)) return false; }
  else if (!fix(g.a_ks, g.a_gs, K, M, d.ra)) return false;
  if (g.b_ks == 1) { if (!fix(g.b_ns, g.b_gs, N, K, d.rb)) return false; }
  else if (!fix(g.b_ks, g.b_gs, K, N, d.rb)) return false;
  return gemm16_plan(g, true);
}

// ---------------------------------------------------------------------------
// pass 1: inlining and pass-through removal
// ---------------------------------------------------------------------------
struct Inliner {
  Module& m;
  std::map<Value*, Value*> remap;
  int depth = 0;
  explicit Inliner(Module& mod) : m(mod) {}

  Value* res(Value* v) {
    auto it = remap.find(v);
    while (it != remap.end()) { v = it->second; it = remap.find(v); }
    return v;
  }

  std::unique_ptr<Op> clone_op(Op* src, std::map<Value*, Value*>& vm) {
    auto op = std::make_unique<Op>();
    op->name = src->name;
    op->attrs = src->attrs;
    for (auto* o : src->operands) {
      auto it = vm.find(o);
      op->operands.push_back(it == vm.end() ? o : it->second);
    }
    for (auto* r : src->results) {
      Value* nv = m.new_value(r->type, r->name);
      nv->def = op.get();
      nv->def_index = r->def_index;
      vm[r] = nv;
      op->results.push_back(nv);
    }
    for (auto& reg : src->regions) {
      auto b = std::make_unique<Block>();
      b->parent_op = op.get();
      for (auto* a : reg->args) {
        Value* nv = m.new_value(a->type, a->name);
        nv->owner = b.get();
        nv->arg_index = a->arg_index;
        vm[a] = nv;
        b->args.push_back(nv);
      }
      for (auto& inner : reg->ops) {
        auto c = clone_op(inner.get(), vm);
        c->parent = b.get();
        b->ops.push_back(std::move(c));
      }
      op->regions.push_back(std::move(b));
    }
    return op;
  }

  void run(Block* b) {
    std::vector<std::unique_ptr<Op>> in = std::move(b->ops);
    b->ops.clear();
    for (auto& op : in) process(std::move(op), b);
  }

  void process(std::unique_ptr<Op> op, Block* b) {
    for (auto& o : op->operands) o = res(o);
    std::string sh = op->short_name();
    // A composite that names a chlo operation this compiler has itself (unary mathematics, atan2, top_k) is that
    // operation; any other composite is its decomposition (src/pjrt_plugin/ops/control_flow.cc:2206-2250).
    if (sh == "composite" && op->has("name")) {
      const std::string cname = attr_str(op->attr("name"));
      if (cname.rfind("chlo.", 0) == 0) {
        const std::string fn = cname.substr(5);
        const bool same = !op->results.empty() && !op->operands.empty() && op->operands[0]->type == op->results[0]->type;
        const bool unary = op->operands.size() == 1 && op->results.size() == 1 && same && is_elementwise_op(fn) && dt_is_float(op->results[0]->type.dt);
        const bool atan2 = fn == "atan2" && op->operands.size() == 2 && op->results.size() == 1 && same && op->operands[1]->type == op->results[0]->type;
        const bool topk = fn == "top_k" && op->operands.size() == 1 && op->results.size() == 2;
        if (unary || atan2 || topk) {
          op->name = atan2 ? "stablehlo.atan2" : cname;
          op->attrs.clear();
          process(std::move(op), b);
          return;
        }
      }
    }
    if (op->name == "func.call" || sh == "composite") {
      std::string callee = attr_str(op->attr(sh == "composite" ? "decomposition" : "callee"));
      if (!callee.empty() && callee[0] == '@') callee = callee.substr(1);
      auto it = m.funcs.find(callee);
      if (it == m.funcs.end()) throw CompileError("call to unknown function @" + callee);
      if (++depth > 64) throw CompileError("call depth limit (recursive functions are not supported)");
      Func* f = it->second.get();
      std::map<Value*, Value*> vm;
      if (f->body->args.size() != op->operands.size()) throw CompileError("call arity mismatch for @" + callee);
      for (size_t k = 0; k < op->operands.size(); k++) vm[f->body->args[k]] = op->operands[k];
      for (auto& inner : f->body->ops) {
        if (inner->name == "func.return") {
          for (size_t k = 0; k < op->results.size(); k++) {
            Value* r = inner->operands[k];
            auto f2 = vm.find(r);
            remap[op->results[k]] = res(f2 == vm.end() ? r : f2->second);
          }
          break;
        }
        auto c = clone_op(inner.get(), vm);
        process(std::move(c), b);
      }
      depth--;
      return;
    }
    if (sh == "optimization_barrier") {
      for (size_t k = 0; k < op->results.size(); k++) remap[op->results[k]] = op->operands[k];
      return;
    }
    if (sh == "custom_call") {
      std::string tgt = attr_str(op->attr("call_target_name"));
      // Pass-through targets of SPMD-lowered programs (src/pjrt_plugin/ops/control_flow.cc:1426-1438).
      if (tgt == "Sharding" || tgt == "SPMDFullToShardShape" || tgt == "SPMDShardToFullShape") {
        if (op->operands.size() == 1 && op->results.size() == 1 && op->operands[0]->type == op->results[0]->type) {
          remap[op->results[0]] = op->operands[0];
          return;
        }
        throw CompileError("custom_call @" + tgt + " that changes the shape needs an SPMD partitioner; "
                           "compile the per-shard (manual) program instead");
      }
      // Unary mathematics and top-k that jax emits as custom calls (src/pjrt_plugin/ops/control_flow.cc:1440-1477): the
      // same operations as their chlo forms.
      if (tgt.rfind("mhlo.", 0) == 0 && op->operands.size() == 1) {
        const std::string fn = tgt.substr(5);
        if (op->results.size() == 1 && is_elementwise_op(fn) && op->operands[0]->type == op->results[0]->type) {
          op->name = "chlo." + fn;
          op->attrs.clear();
          process(std::move(op), b);
          return;
        }
        if (fn == "topk" && op->results.size() == 2) {
          op->name = "chlo.top_k";
          op->attrs.clear();
          process(std::move(op), b);
          return;
        }
      }
    }
    // convert(convert(x, wider type), type of x) -> x when the first conversion is exact (bf16 -> f32 -> bf16 between two
    // products of a bf16 network)
    if (sh == "convert" && op->operands.size() == 1 && op->operands[0]->def && op->operands[0]->def->short_name() == "convert") {
      Value* inner = op->operands[0]->def->operands[0];
      const DT a = inner->type.dt, mid = op->operands[0]->type.dt;
      auto widens = [](DT from, DT to) {
        if ((from == DT::BF16 || from == DT::F16) && (to == DT::F32 || to == DT::F64)) return true;
        if (from == DT::F32 && to == DT::F64) return true;
        if (dt_is_signed(from) && dt_is_signed(to) && dt_size(to) > dt_size(from)) return true;
        if (dt_is_unsigned(from) && dt_is_int(to) && dt_size(to) > dt_size(from)) return true;
        return false;
      };
      if (inner->type == op->results[0]->type && widens(a, mid)) {
        remap[op->results[0]] = res(inner);
        return;
      }
    }
    // the same round trip through a reshape: convert(reshape(convert(x))) back to x's type is reshape(x), a view
    if (sh == "convert" && op->operands.size() == 1 && op->operands[0]->def && op->operands[0]->def->short_name() == "reshape" &&
        op->operands[0]->def->operands[0]->def && op->operands[0]->def->operands[0]->def->short_name() == "convert") {
      Op* inner_cv = op->operands[0]->def->operands[0]->def;
      Value* inner = inner_cv->operands[0];
      const DT a = inner->type.dt, mid = inner_cv->results[0]->type.dt;
      const bool widens = (a == DT::BF16 || a == DT::F16) && (mid == DT::F32 || mid == DT::F64);
      if (widens && op->results[0]->type.dt == a && inner->type.numel() == op->results[0]->type.numel()) {
        op->name = "stablehlo.reshape";
        op->attrs.clear();
        op->operands = {res(inner)};
        sh = "reshape";
      }
    }
    // x + broadcast(0), x * broadcast(1), x - broadcast(0), x / broadcast(1) -> x
    // (src/pjrt_plugin/passes/canonicalize_broadcast_identity.cc)
    if ((sh == "add" || sh == "multiply" || sh == "subtract" || sh == "divide") && op->operands.size() == 2 &&
        dt_is_float(op->results[0]->type.dt)) {
      auto splat_of = [&](Value* v, double& out) -> bool {
        Op* d = v->def;
        while (d && (d->short_name() == "broadcast_in_dim" || d->short_name() == "reshape")) d = d->operands[0]->def;
        if (!d || d->short_name() != "constant") return false;
        DenseValue dv = attr_dense(d->attr("value"));
        if (!dv.splat || dv.type.numel() == 0) return false;
        if (dv.type.dt == DT::F32) { float f; memcpy(&f, dv.data.data(), 4); out = f; return true; }
        if (dv.type.dt == DT::BF16) { uint16_t h; memcpy(&h, dv.data.data(), 2); out = bf16_to_f32(h); return true; }
        return false;
      };
      double c;
      double ident = (sh == "add" || sh == "subtract") ? 0.0 : 1.0;
      auto is_ident = [&](double x) { return x == ident && !(ident == 0.0 && std::signbit(x)); };
      if (splat_of(op->operands[1], c) && is_ident(c) && op->operands[0]->type == op->results[0]->type) {
        remap[op->results[0]] = op->operands[0];
        return;
      }
      if ((sh == "add" || sh == "multiply") && splat_of(op->operands[0], c) && is_ident(c) &&
          op->operands[1]->type == op->results[0]->type) {
        remap[op->results[0]] = op->operands[1];
        return;
      }
    }
    // convolution whose kernel is a stablehlo.reverse over kernel-spatial dimensions (the input gradient of a
    // convolution): the reversal is folded into the B index table instead of materialising the flipped kernel
    if (sh == "convolution" && op->operands.size() == 2 && op->operands[1]->def &&
        op->operands[1]->def->short_name() == "reverse" && !op->has("b200.rhs_reversed")) {
      Op* rev = op->operands[1]->def;
      const std::string& dn = op->attr("dimension_numbers");
      size_t a1 = dn.find(']'), b0 = dn.find('[', a1), b1 = dn.find(']', b0);
      if (a1 != std::string::npos && b0 != std::string::npos && b1 != std::string::npos) {
        std::vector<int64_t> spatial;          // kernel dimensions labelled with a digit
        int64_t d = 0;
        std::string cur;
        for (size_t k = b0 + 1; k <= b1; k++) {
          char ch = dn[k];
          if (ch == ',' || ch == ']') {
            if (!cur.empty() && isdigit((unsigned char)cur[0])) spatial.push_back(d);
            cur.clear();
            d++;
          } else if (!isspace((unsigned char)ch)) cur += ch;
        }
        std::vector<int64_t> rd = attr_i64s(rev->attr("dimensions"));
        bool ok = !rd.empty();
        for (auto x : rd) ok = ok && std::find(spatial.begin(), spatial.end(), x) != spatial.end();
        if (ok) {
          std::string txt = "[";
          for (size_t k = 0; k < rd.size(); k++) txt += (k ? ", " : "") + std::to_string(rd[k]);
          op->attrs["b200.rhs_reversed"] = txt + "]";
          op->operands[1] = res(rev->operands[0]);
        }
      }
    }
    // Convolutions whose innermost input dimension is a small channel count that is not a multiple of four (an RGB
    // stem, forward and weight gradient) cannot be gathered 16 bytes at a time. The input is zero-padded to four
    // channels (and the kernel's input-feature dimension with it, or the weight gradient sliced back), which moves
    // them from the scalar-gather kernel to the vector paths.
    if (sh == "convolution" && op->operands.size() == 2 && op->results.size() == 1 &&
        (!op->has("feature_group_count") || attr_int(op->attr("feature_group_count")) == 1) &&
        (!op->has("batch_group_count") || attr_int(op->attr("batch_group_count")) == 1)) {
      const std::string& dn = op->attr("dimension_numbers");
      auto spec = [&](size_t from, size_t& end) {
        std::vector<std::string> toks;
        size_t b0 = dn.find('[', from), b1 = dn.find(']', b0);
        end = b1;
        if (b0 == std::string::npos || b1 == std::string::npos) return toks;
        std::string cur;
        for (size_t k = b0 + 1; k <= b1; k++) {
          if (dn[k] == ',' || dn[k] == ']') { toks.push_back(cur); cur.clear(); }
          else if (!isspace((unsigned char)dn[k])) cur += dn[k];
        }
        return toks;
      };
      size_t e1 = 0, e2 = 0, e3 = 0;
      auto ls = spec(0, e1);
      auto rs = e1 != std::string::npos ? spec(e1, e2) : std::vector<std::string>{};
      auto os = e2 != std::string::npos ? spec(e2, e3) : std::vector<std::string>{};
      auto pos = [](const std::vector<std::string>& v, const char* c) { for (size_t k = 0; k < v.size(); k++) if (v[k] == c) return (int)k; return -1; };
      Value *lhs = op->operands[0], *rhs = op->operands[1];
      const int rank = lhs->type.rank();
      const int lb = pos(ls, "b"), lf = pos(ls, "f"), ri = pos(rs, "i"), ob = pos(os, "b");
      auto pad_dim = [&](Value* v, int dim, int64_t to) -> Value* {
        auto key = std::make_tuple(v, dim, to);
        auto it = padded.find(key);
        if (it != padded.end()) return it->second;
        TensorType st;
        st.dt = v->type.dt;
        auto zc = std::make_unique<Op>();
        zc->name = "stablehlo.constant";
        zc->attrs["value"] = "dense<0.000000e+00> : " + st.str();
        Value* zero = m.new_value(st, "");
        zero->def = zc.get();
        zero->def_index = 0;
        zc->results.push_back(zero);
        zc->parent = b;
        b->ops.push_back(std::move(zc));
        auto pd = std::make_unique<Op>();
        pd->name = "stablehlo.pad";
        pd->operands = {v, zero};
        std::string lo = "array<i64: ", hi = "array<i64: ";
        for (int k = 0; k < v->type.rank(); k++) {
          lo += std::string(k ? ", " : "") + "0";
          hi += std::string(k ? ", " : "") + std::to_string(k == dim ? to - v->type.dims[k] : 0);
        }
        pd->attrs["edge_padding_low"] = lo + ">";
        pd->attrs["edge_padding_high"] = hi + ">";
        pd->attrs["interior_padding"] = lo + ">";
        TensorType pt = v->type;
        pt.dims[dim] = to;
        Value* out = m.new_value(pt, "");
        out->def = pd.get();
        out->def_index = 0;
        pd->results.push_back(out);
        pd->parent = b;
        b->ops.push_back(std::move(pd));
        padded[key] = out;
        return out;
      };
      if (rank >= 3 && lb >= 0 && lf >= 0 && ri >= 0 && ob >= 0 && (int)ls.size() == rank && dt_is_float(lhs->type.dt)) {
        const int64_t Cin = lhs->type.dims[lf], Nb = lhs->type.dims[lb];
        if (lf == rank - 1 && Cin % 4 != 0 && Cin < 16 && rhs->type.dims[ri] == Cin) {
          const int64_t to = (Cin + 3) / 4 * 4;
          op->operands[0] = pad_dim(lhs, lf, to);
          op->operands[1] = pad_dim(rhs, ri, to);
        } else if (lb == rank - 1 && Nb % 4 != 0 && Nb < 16 && op->results[0]->type.dims[ob] == Nb) {
          const int64_t to = (Nb + 3) / 4 * 4;
          op->operands[0] = pad_dim(lhs, lb, to);
          // the convolution now yields `to` slices along the output's batch dimension; the first Nb are the result
          Value* orig = op->results[0];
          TensorType wt = orig->type;
          wt.dims[ob] = to;
          Value* wide = m.new_value(wt, "");
          wide->def = op.get();
          wide->def_index = 0;
          op->results[0] = wide;
          auto sl = std::make_unique<Op>();
          sl->name = "stablehlo.slice";
          sl->operands = {wide};
          std::string st0 = "array<i64: ", lim = "array<i64: ", one = "array<i64: ";
          for (int k = 0; k < orig->type.rank(); k++) {
            st0 += std::string(k ? ", " : "") + "0";
            lim += std::string(k ? ", " : "") + std::to_string(orig->type.dims[k]);
            one += std::string(k ? ", " : "") + "1";
          }
          sl->attrs["start_indices"] = st0 + ">";
          sl->attrs["limit_indices"] = lim + ">";
          sl->attrs["strides"] = one + ">";
          orig->def = sl.get();
          orig->def_index = 0;
          sl->results.push_back(orig);
          deferred.push_back(std::move(sl));
        }
      }
    }
    // dot_general on integers and booleans: exact integer arithmetic (wrapping like any integer multiply and add; the
    // reference casts through f32, src/pjrt_plugin/ops/linalg.cc:110-119, which is exact only below 2^24). The product
    // is written as what it means, result[b, i, j] = sum over k of lhs[b, i, k] * rhs[b, k, j]: both operands broadcast
    // to [batch, lhs free, rhs free, contracted], multiplied and reduced over the trailing dimensions. The broadcasts
    // and the multiply are evaluated inside the reduction kernel; nothing of the large shape is stored.
    // chlo.top_k (src/pjrt_plugin/ops/sort_fft_complex.cc:41-88): a stable descending sort of the values together with
    // their positions along the last dimension, of which the first k are kept. NaN goes after every number.
    if (op->name == "chlo.top_k" && op->operands.size() == 1 && op->results.size() == 2) {
      Value* x = op->operands[0];
      const TensorType xt = x->type;
      const int R = xt.rank();
      if (R < 1) throw CompileError("chlo.top_k of a scalar");
      const int64_t kk = op->results[0]->type.dims.empty() ? 0 : op->results[0]->type.dims.back();
      auto make = [&](const std::string& name, std::vector<Value*> ins, std::vector<Value*> outs, std::map<std::string, std::string> attrs) {
        auto o = std::make_unique<Op>();
        o->name = name;
        o->operands = std::move(ins);
        o->attrs = std::move(attrs);
        for (size_t q = 0; q < outs.size(); q++) { outs[q]->def = o.get(); outs[q]->def_index = (int)q; o->results.push_back(outs[q]); }
        return o;
      };
      TensorType it = xt;
      it.dt = DT::I32;
      Value* pos = m.new_value(it, "");
      process(make("stablehlo.iota", {}, {pos}, {{"iota_dimension", std::to_string(R - 1) + " : i64"}}), b);
      Value* sv = m.new_value(xt, "");
      Value* sp = m.new_value(it, "");
      auto sort = make("stablehlo.sort", {x, res(pos)}, {sv, sp}, {{"dimension", std::to_string(R - 1) + " : i64"}, {"is_stable", "true"}});
      auto body = std::make_unique<Block>();
      body->parent_op = sort.get();
      TensorType st, bt, pt;
      st.dt = xt.dt;
      bt.dt = DT::PRED;
      pt.dt = DT::I32;
      Value* args[4] = {m.new_value(st, "%a"), m.new_value(st, "%b"), m.new_value(pt, "%pa"), m.new_value(pt, "%pb")};
      for (Value* v : args) { v->owner = body.get(); v->arg_index = (int)body->args.size(); body->args.push_back(v); }
      auto inner = [&](const std::string& name, std::vector<Value*> ins, std::map<std::string, std::string> attrs) {
        Value* r = m.new_value(bt, "");
        auto o = make(name, std::move(ins), {r}, std::move(attrs));
        o->parent = body.get();
        body->ops.push_back(std::move(o));
        return r;
      };
      auto cmp = [&](Value* l, Value* r, const char* dir) {
        const char* ct = dt_is_float(xt.dt) ? "FLOAT" : (dt_is_unsigned(xt.dt) || xt.dt == DT::PRED ? "UNSIGNED" : "SIGNED");
        return inner("stablehlo.compare", {l, r}, {{"comparison_direction", std::string("#stablehlo<comparison_direction ") + dir + ">"},
                                                    {"compare_type", std::string("#stablehlo<comparison_type ") + ct + ">"}});
      };
      Value* first = cmp(args[0], args[1], "GT");
      if (dt_is_float(xt.dt)) {
        Value* b_nan = cmp(args[1], args[1], "NE");
        Value* a_num = cmp(args[0], args[0], "EQ");
        first = inner("stablehlo.or", {first, inner("stablehlo.and", {b_nan, a_num}, {})}, {});
      }
      auto ret = std::make_unique<Op>();
      ret->name = "stablehlo.return";
      ret->operands = {first};
      ret->parent = body.get();
      body->ops.push_back(std::move(ret));
      sort->regions.push_back(std::move(body));
      process(std::move(sort), b);
      std::string zeros = "array<i64", lim = "array<i64", ones = "array<i64";
      for (int d = 0; d < R; d++) {
        zeros += (d ? ", 0" : ": 0");
        ones += (d ? ", 1" : ": 1");
        lim += (d ? ", " : ": ") + std::to_string(d == R - 1 ? kk : xt.dims[d]);
      }
      zeros += ">"; ones += ">"; lim += ">";
      for (int q = 0; q < 2; q++)
        process(make("stablehlo.slice", {res(q == 0 ? sv : sp)}, {op->results[q]}, {{"start_indices", zeros}, {"limit_indices", lim}, {"strides", ones}}), b);
      return;
    }
    if (sh == "dot_general" && op->operands.size() == 2 && op->results.size() == 1 && op->has("dot_dimension_numbers")) {
      auto integral = [](DT d) { return d == DT::PRED || dt_is_signed(d) || dt_is_unsigned(d); };
      const TensorType rt = op->results[0]->type;
      if (integral(rt.dt) && integral(op->operands[0]->type.dt) && integral(op->operands[1]->type.dt)) {
        auto f = attr_struct(op->attr("dot_dimension_numbers"));
        const auto lb = f["lhs_batching_dimensions"], rb = f["rhs_batching_dimensions"];
        const auto lc = f["lhs_contracting_dimensions"], rc = f["rhs_contracting_dimensions"];
        Value* ops2[2] = {op->operands[0], op->operands[1]};
        auto new_op = [&](const char* name, std::vector<Value*> ins, const TensorType& t, std::map<std::string, std::string> attrs,
                          Value* into = nullptr) -> std::unique_ptr<Op> {
          auto o = std::make_unique<Op>();
          o->name = std::string("stablehlo.") + name;
          o->operands = std::move(ins);
          o->attrs = std::move(attrs);
          Value* v = into ? into : m.new_value(t, "");
          v->def = o.get();
          v->def_index = 0;
          o->results.push_back(v);
          return o;
        };
        auto run1 = [&](std::unique_ptr<Op> o) -> Value* {
          Value* v = o->results[0];
          process(std::move(o), b);
          return res(v);
        };
        auto pos_in = [](const std::vector<int64_t>& v, int64_t x) { for (size_t k = 0; k < v.size(); k++) if (v[k] == x) return (int)k; return -1; };
        std::vector<int64_t> full = rt.dims;
        for (auto d : lc) full.push_back(ops2[0]->type.dims[d]);
        const int nb = (int)lb.size(), nres = (int)rt.dims.size();
        int nlf = 0;
        for (int d = 0; d < ops2[0]->type.rank(); d++) if (pos_in(lb, d) < 0 && pos_in(lc, d) < 0) nlf++;
        Value* wide[2];
        for (int side = 0; side < 2; side++) {
          Value* v = ops2[side];
          const auto& bd = side == 0 ? lb : rb;
          const auto& cd = side == 0 ? lc : rc;
          if (v->type.dt != rt.dt) {
            TensorType ct = v->type;
            ct.dt = rt.dt;
            v = run1(new_op("convert", {v}, ct, {}));
          }
          std::string map = "[";
          int free_seen = 0;
          for (int d = 0; d < v->type.rank(); d++) {
            int to;
            if (pos_in(bd, d) >= 0) to = pos_in(bd, d);
            else if (pos_in(cd, d) >= 0) to = nres + pos_in(cd, d);
            else to = nb + (side == 0 ? 0 : nlf) + free_seen++;
            map += (d ? ", " : "") + std::to_string(to);
          }
          map += "]";
          TensorType ft;
          ft.dt = rt.dt;
          ft.dims = full;
          wide[side] = run1(new_op("broadcast_in_dim", {v}, ft, {{"broadcast_dimensions", map}}));
        }
        TensorType ft;
        ft.dt = rt.dt;
        ft.dims = full;
        const bool boolean = rt.dt == DT::PRED;
        if (lc.empty()) {
          process(new_op(boolean ? "and" : "multiply", {wide[0], wide[1]}, rt, {}, op->results[0]), b);
          return;
        }
        Value* prod = run1(new_op(boolean ? "and" : "multiply", {wide[0], wide[1]}, ft, {}));
        TensorType st;
        st.dt = rt.dt;
        Value* init = run1(new_op("constant", {}, st, {{"value", std::string("dense<") + (boolean ? "false" : "0") + "> : " + st.str()}}));
        std::string dims = "[";
        for (size_t k = 0; k < lc.size(); k++) dims += (k ? ", " : "") + std::to_string(nres + (int)k);
        dims += "]";
        auto red = new_op("reduce", {prod, init}, rt, {{"dimensions", dims}}, op->results[0]);
        auto body = std::make_unique<Block>();
        body->parent_op = red.get();
        Value* a0 = m.new_value(st, "%acc");
        Value* a1 = m.new_value(st, "%val");
        for (Value* v : {a0, a1}) { v->owner = body.get(); v->arg_index = (int)body->args.size(); body->args.push_back(v); }
        auto inner = std::make_unique<Op>();
        inner->name = boolean ? "stablehlo.or" : "stablehlo.add";
        inner->operands = {a0, a1};
        inner->parent = body.get();
        Value* r = m.new_value(st, "%red");
        r->def = inner.get();
        inner->results.push_back(r);
        auto ret = std::make_unique<Op>();
        ret->name = "stablehlo.return";
        ret->operands = {r};
        ret->parent = body.get();
        body->ops.push_back(std::move(inner));
        body->ops.push_back(std::move(ret));
        red->regions.push_back(std::move(body));
        process(std::move(red), b);
        return;
      }
    }
    // dot_general on two bf16 (or two f16) operands in matrix form goes to the native 16-bit kernels (lower_dot16).
    // Any other dot_general / convolution on bf16 or f16 operands: computed as the f32 contraction of the converted
    // operands and rounded once at the end. Products of two bf16 (or f16) numbers and their fp32 accumulation
    // are what XLA's CPU backend computes for these types; the converts fuse into neighbouring kernels.
    if ((sh == "dot_general" || sh == "convolution") && op->operands.size() == 2 && op->results.size() == 1) {
      auto half = [](DT d) { return d == DT::BF16 || d == DT::F16; };
      Dot16 native;
      const bool is_native = sh == "dot_general" && dot16_geometry(op.get(), native);
      if (!is_native && (half(op->operands[0]->type.dt) || half(op->operands[1]->type.dt) || half(op->results[0]->type.dt))) {
        auto convert_to = [&](Value* v, DT to, Value* into) -> Value* {
          // The widened copy of an operand that comes from outside a `while` (weights read by a decode loop) is
          // made once in front of the loop instead of in every iteration: the convert moves out through every
          // enclosing loop region that does not define the operand.
          Block* tb = b;
          if (!into && !getenv("B200_NO_HOIST")) {
            for (size_t lvl = enclosing.size(); lvl-- > 0;) {
              auto& en = enclosing[lvl];
              const bool defined_here = v->def ? v->def->parent == tb : v->owner == tb;
              if (defined_here || en.second->short_name() != "while") break;
              bool is_region = false;
              for (auto& reg : en.second->regions) is_region = is_region || reg.get() == tb;
              if (!is_region) break;
              tb = en.first;
            }
            if (tb != b) {
              auto hit = hoisted.find({v, (int)to});
              if (hit != hoisted.end()) return hit->second;
            }
          }
          auto c = std::make_unique<Op>();
          c->name = "stablehlo.convert";
          c->operands.push_back(v);
          TensorType t = v->type;
          t.dt = to;
          Value* nv = into ? into : m.new_value(t, "");
          nv->def = c.get();
          nv->def_index = 0;
          c->results.push_back(nv);
          c->parent = tb;
          tb->ops.push_back(std::move(c));
          if (tb != b) hoisted[{v, (int)to}] = nv;
          return nv;
        };
        for (auto& o : op->operands)
          if (half(o->type.dt)) o = convert_to(o, DT::F32, nullptr);
        Value* orig = op->results[0];
        if (half(orig->type.dt)) {
          TensorType t = orig->type;
          t.dt = DT::F32;
          Value* wide = m.new_value(t, "");
          wide->def = op.get();
          wide->def_index = 0;
          op->results[0] = wide;
          op->parent = b;
          b->ops.push_back(std::move(op));
          convert_to(wide, orig->type.dt, orig);
          for (auto& d : deferred) { d->parent = b; b->ops.push_back(std::move(d)); }
          deferred.clear();
          return;
        }
      }
    }
    // Common subexpressions: an operation without regions or side effects that repeats an earlier one of the same
    // block (same name, operands, attributes and result types) is dropped and its results renamed. Generators and
    // jax alike emit the same convert or broadcast once per use (the bf16 copy of a normalised activation feeding
    // three projections); without this every copy becomes its own kernel launch.
    if (op->regions.empty() && deferred.empty() && cse_candidate(op.get())) {
      std::string key = op->name;
      for (auto* o : op->operands) { char buf[32]; snprintf(buf, sizeof buf, "|%p", (void*)o); key += buf; }
      for (auto& kv : op->attrs) key += "|" + kv.first + "=" + kv.second;
      for (auto* r : op->results) key += "|" + r->type.str();
      auto& table = seen_ops[b];
      auto it = table.find(key);
      if (it != table.end()) {
        for (size_t k = 0; k < op->results.size(); k++) remap[op->results[k]] = it->second->results[k];
        return;
      }
      table[key] = op.get();
    }
    enclosing.push_back({b, op.get()});
    for (auto& reg : op->regions) run(reg.get());
    enclosing.pop_back();
    op->parent = b;
    b->ops.push_back(std::move(op));
    for (auto& d : deferred) { d->parent = b; b->ops.push_back(std::move(d)); }
    deferred.clear();
  }
  static bool cse_candidate(Op* op) {
    if (getenv("B200_NO_CSE")) return false;
    const std::string sh = op->short_name();
    if (op->name.rfind("stablehlo.", 0) != 0 && op->name.rfind("chlo.", 0) != 0) return false;
    if (is_elementwise_op(sh)) return true;
    static const char* pure[] = {"broadcast_in_dim", "reshape", "transpose", "reverse", "slice", "pad", "concatenate", "dynamic_slice",
                                 "iota", "gather", "dot_general", "convolution", "convert", "bitcast_convert", "dynamic_update_slice"};
    for (const char* p2 : pure) if (sh == p2) return true;
    return false;
  }
  std::map<Block*, std::map<std::string, Op*>> seen_ops;         // per block: key of an operation -> its first occurrence
  std::vector<std::pair<Block*, Op*>> enclosing;               // (block, op) pairs around the region being processed
  std::map<std::pair<Value*, int>, Value*> hoisted;            // widened copies already placed in front of a loop
  std::map<std::tuple<Value*, int, int64_t>, Value*> padded;   // zero-padded copies made for convolutions
  std::vector<std::unique_ptr<Op>> deferred;                   // ops to place right after the one being processed
};

void fix_region_operands(Block* b, Inliner& inl) {
  for (auto& op : b->ops) {
    for (auto& o : op->operands) o = inl.res(o);
    for (auto& r : op->regions) fix_region_operands(r.get(), inl);
  }
}

// ---------------------------------------------------------------------------
// pass 1b: weights of skinny products inside loops
// ---------------------------------------------------------------------------
// A decode loop multiplies one or a few rows by weight matrices that come from outside the loop, once per iteration:
// the rate is the rate at which the weights stream from HBM. A 16-bit weight stored [k][n] (n contiguous) needs a K
// split across CTAs to give the GPU enough independent loads, and the split costs a reduction pass; stored [n][k]
// every output column is one contiguous row that a warp streams with 128-bit loads and finishes with a shuffle tree.
// So for every such product the transposed weight is made once in front of the loop, and products that share their
// left operand (the query / key / value projections, the gate and up projections) read one concatenated weight and
// become one product whose result is sliced. What it costs: one pass over the weights per execution and a second
// copy of them in HBM.
struct SkinnyWeightHoist {
  Module& m;
  explicit SkinnyWeightHoist(Module& mod) : m(mod) {}

  static std::string i64_array(const std::vector<int64_t>& v) {
    std::string s = "array<i64: ";
    for (size_t k = 0; k < v.size(); k++) s += (k ? ", " : "") + std::to_string(v[k]);
    return s + ">";
  }
  Value* make(std::unique_ptr<Op>& op, const TensorType& t, Block* parent) {
    Value* v = m.new_value(t, "");
    v->def = op.get();
    v->def_index = 0;
    op->results.push_back(v);
    op->parent = parent;
    return v;
  }
  static bool defined_in(Value* v, Block* b) {
    if (v->def) {
      for (Block* p = v->def->parent; p; p = p->parent_op ? p->parent_op->parent : nullptr)
        if (p == b) return true;
      return false;
    }
    for (Block* p = v->owner; p; p = p->parent_op ? p->parent_op->parent : nullptr)
      if (p == b) return true;
    return false;
  }

  void run(Block* b) {
    for (size_t i = 0; i < b->ops.size(); i++) {
      Op* op = b->ops[i].get();
      for (auto& r : op->regions) run(r.get());
      if (op->short_name() != "while" || op->regions.size() != 2 || getenv("B200_NO_WEIGHT_HOIST")) continue;
      std::vector<std::unique_ptr<Op>> front;          // operations to place in front of the loop
      hoist_invariants(op->regions[1].get(), b, front);
      rewrite(op->regions[1].get(), b, front);
      const size_t n = front.size();
      for (size_t k = 0; k < n; k++) b->ops.insert(b->ops.begin() + i + k, std::move(front[k]));
      i += n;
    }
  }

  // Loop-invariant code motion: a pure elementwise or indexing operation of the body whose operands all come from
  // outside the loop (or from operations moved before it) is computed once in front of the loop: the (1 + w) scale of
  // every norm of a decode loop, a mask built from constants. Constants, iotas and broadcasts stay where they are (their
  // users evaluate them inline for free) and are copied in front of the loop only where a moved operation needs them.
  void hoist_invariants(Block* body, Block* outer, std::vector<std::unique_ptr<Op>>& front) {
    if (getenv("B200_NO_LICM")) return;
    std::set<Value*> moved;                           // results now defined in front of the loop
    std::map<Op*, Value*> dup_copy;                   // duplicable operations copied in front of the loop
    std::function<bool(Value*, int)> invariant = [&](Value* v, int depth) -> bool {
      if (moved.count(v) || !defined_in(v, body)) return true;
      Op* d = v->def;
      if (!d || d->parent != body || depth > 8) return false;
      const std::string sh = d->short_name();
      if (sh == "constant" || sh == "iota") return true;
      if (sh == "broadcast_in_dim") return invariant(d->operands[0], depth + 1);
      return false;
    };
    std::function<Value*(Value*)> outside = [&](Value* v) -> Value* {
      if (moved.count(v) || !defined_in(v, body)) return v;
      Op* d = v->def;                                 // a constant, iota or broadcast: copy it
      auto it = dup_copy.find(d);
      if (it != dup_copy.end()) return it->second;
      auto c = std::make_unique<Op>();
      c->name = d->name;
      c->attrs = d->attrs;
      for (Value* o : d->operands) c->operands.push_back(outside(o));
      Value* nv = make(c, v->type, outer);
      front.push_back(std::move(c));
      dup_copy[d] = nv;
      return nv;
    };
    std::vector<std::unique_ptr<Op>> kept;
    for (auto& up : body->ops) {
      Op* op = up.get();
      const std::string sh = op->short_name();
      static const std::set<std::string> indexing = {"reshape", "transpose", "reverse", "slice", "pad", "concatenate", "convert"};
      const bool pure = op->regions.empty() && op->results.size() == 1 && (op->name.rfind("stablehlo.", 0) == 0) &&
                        (is_elementwise_op(sh) || indexing.count(sh));
      bool ok = pure && !op->operands.empty() && op->results[0]->type.numel() <= (1 << 24);
      bool any_real = false;                          // reads something that is not a constant: worth a kernel of its own
      for (Value* o : op->operands) {
        ok = ok && invariant(o, 0);
        any_real = any_real || moved.count(o) || !defined_in(o, body);
      }
      if (!ok || !any_real) { kept.push_back(std::move(up)); continue; }
      for (auto& o : op->operands) o = outside(o);
      op->parent = outer;
      moved.insert(op->results[0]);
      front.push_back(std::move(up));
    }
    body->ops = std::move(kept);
  }

  void rewrite(Block* body, Block* outer, std::vector<std::unique_ptr<Op>>& front) {
    struct Cand { Op* op; Value* lhs; Value* rhs; int64_t K, N; };
    std::map<Value*, std::vector<Cand>> by_lhs;
    std::vector<Value*> order;
    for (auto& up : body->ops) {
      Op* op = up.get();
      if (op->short_name() != "dot_general" || op->operands.size() != 2 || !op->has("dot_dimension_numbers")) continue;
      Value *lhs = op->operands[0], *rhs = op->operands[1];
      const DT dt = lhs->type.dt;
      if (dt != rhs->type.dt || !(dt == DT::BF16 || dt == DT::F16) || rhs->type.rank() != 2 || lhs->type.rank() < 1) continue;
      if (defined_in(rhs, body)) continue;             // not loop-invariant
      auto f = attr_struct(op->attr("dot_dimension_numbers"));
      if (!f["lhs_batching_dimensions"].empty() || !f["rhs_batching_dimensions"].empty()) continue;
      auto lcd = f["lhs_contracting_dimensions"], rcd = f["rhs_contracting_dimensions"];
      if (lcd.size() != 1 || rcd.size() != 1 || lcd[0] != lhs->type.rank() - 1 || rcd[0] != 0) continue;
      const int64_t K = rhs->type.dims[0], N = rhs->type.dims[1];
      const int64_t M = lhs->type.numel() / std::max<int64_t>(K, 1);
      if (M > 8 || K % 8 || K * N < (1 << 16) || M * K * 2 > 96 * 1024) continue;
      if (!by_lhs.count(lhs)) order.push_back(lhs);
      by_lhs[lhs].push_back({op, lhs, rhs, K, N});
    }
    for (Value* lhs : order) {
      auto& group = by_lhs[lhs];
      // transposed (and concatenated) weight in front of the loop
      std::vector<Value*> parts;
      int64_t total = 0;
      const int64_t K = group[0].K;
      for (auto& c : group) {
        auto key = std::make_pair(c.rhs, outer);
        Value* t;
        auto tr = std::make_unique<Op>();
        tr->name = "stablehlo.transpose";
        tr->operands = {c.rhs};
        tr->attrs["permutation"] = i64_array({1, 0});
        TensorType tt = c.rhs->type;
        tt.dims = {c.N, c.K};
        t = make(tr, tt, outer);
        front.push_back(std::move(tr));
        (void)key;
        parts.push_back(t);
        total += c.N;
      }
      Value* weight = parts[0];
      if (parts.size() > 1) {
        auto cat = std::make_unique<Op>();
        cat->name = "stablehlo.concatenate";
        cat->operands = parts;
        cat->attrs["dimension"] = "0 : i64";
        TensorType ct = parts[0]->type;
        ct.dims = {total, K};
        weight = make(cat, ct, outer);
        front.push_back(std::move(cat));
      }
      Op* first = group[0].op;
      const int lrank = lhs->type.rank();
      if (group.size() == 1) {
        // a product on its own keeps its place and result and reads the transposed weight
        first->operands[1] = weight;
        first->attrs["dot_dimension_numbers"] = "#stablehlo.dot<lhs_batching_dimensions = [], rhs_batching_dimensions = [], "
                                                "lhs_contracting_dimensions = [" + std::to_string(lrank - 1) +
                                                "], rhs_contracting_dimensions = [1]>";
        continue;
      }
      // one product against the whole weight, in the place of the group's first product; the others become slices
      std::vector<int64_t> out_dims(lhs->type.dims.begin(), lhs->type.dims.end() - 1);
      out_dims.push_back(total);
      auto dot = std::make_unique<Op>();
      dot->name = "stablehlo.dot_general";
      dot->operands = {lhs, weight};
      dot->attrs = first->attrs;
      dot->attrs["dot_dimension_numbers"] = "#stablehlo.dot<lhs_batching_dimensions = [], rhs_batching_dimensions = [], "
                                            "lhs_contracting_dimensions = [" + std::to_string(lrank - 1) +
                                            "], rhs_contracting_dimensions = [1]>";
      TensorType dt2 = first->results[0]->type;
      dt2.dims = out_dims;
      Value* whole = make(dot, dt2, body);
      // position of the first product in the body
      size_t at = 0;
      while (at < body->ops.size() && body->ops[at].get() != first) at++;
      int64_t off = 0;
      std::vector<std::unique_ptr<Op>> slices;
      for (auto& c : group) {
        // the old product turns into a slice of the new one (same result value, so users need no change)
        Op* old = c.op;
        std::vector<int64_t> st(lrank, 0), lim = out_dims, one(lrank, 1);
        st[lrank - 1] = off;
        lim[lrank - 1] = off + c.N;
        old->name = "stablehlo.slice";
        old->operands = {whole};
        old->attrs.clear();
        old->attrs["start_indices"] = i64_array(st);
        old->attrs["limit_indices"] = i64_array(lim);
        old->attrs["strides"] = i64_array(one);
        off += c.N;
      }
      body->ops.insert(body->ops.begin() + at, std::move(dot));
    }
  }
};

// ---------------------------------------------------------------------------
// Attention over a cache for a handful of queries (a decode step): dot_general(Q, K) -> pointwise (scale, mask) ->
// softmax over the positions -> dot_general(P, V) becomes one operation, `b200.decode_attention`, that keeps the
// pointwise part as a region and is lowered to one kernel (Planner::lower_decode_attention). The reference matches the
// same chain into its fused attention call (src/pjrt_plugin/ops/control_flow.cc:1484-1533 runs it; the matcher is on
// the Python side). Left as it is: anything with more than eight query rows per key / value group, other layouts than
// row-major [groups,] rows x features operands, or intermediate values that something else reads.
// ---------------------------------------------------------------------------
struct DecodeAttentionFusion {
  Module& m;
  explicit DecodeAttentionFusion(Module& mod) : m(mod) {}
  std::map<Value*, int> uses;

  void count(Block* b) {
    for (auto& op : b->ops) {
      for (Value* o : op->operands) uses[o]++;
      for (auto& r : op->regions) count(r.get());
    }
  }
  void run(Block* b) {
    if (getenv("B200_NO_ATTENTION_FUSION")) return;
    uses.clear();
    count(b);
    fuse_in(b);
  }
  void fuse_in(Block* b) {
    for (auto& op : b->ops)
      for (auto& r : op->regions) fuse_in(r.get());
    for (size_t i = 0; i < b->ops.size(); i++)
      if (b->ops[i]->short_name() == "dot_general" && try_fuse(b, b->ops[i].get())) i = (size_t)-1;     // positions changed: start over
  }

  static Op* def_in(Value* v, Block* b, const char* short_name) {
    return v->def && v->def->parent == b && v->def->short_name() == short_name ? v->def : nullptr;
  }
  static bool splat_is(Value* v, double want) {
    Op* d = v->def;
    if (!d || d->short_name() != "constant") return false;
    DenseValue dv = attr_dense(d->attr("value"));
    if (!dv.splat && dv.type.numel() != 1) return false;
    if (dv.type.dt != DT::F32) return false;
    float f;
    memcpy(&f, dv.data.data(), 4);
    return (double)f == want;
  }
  // reduce over the last dimension with a one-operation body
  static bool last_dim_reduce(Op* r, const char* body_op) {
    if (!r || r->operands.size() != 2 || r->results.size() != 1 || r->regions.size() != 1) return false;
    const int rank = r->operands[0]->type.rank();
    auto dims = attr_i64s(r->attr("dimensions"));
    if (dims.size() != 1 || dims[0] != rank - 1) return false;
    Block* body = r->regions[0].get();
    if (body->ops.size() != 2 || body->args.size() != 2 || body->ops[0]->short_name() != body_op) return false;
    Op* c = body->ops[0].get();
    const bool uses_args = (c->operands[0] == body->args[0] && c->operands[1] == body->args[1]) ||
                           (c->operands[0] == body->args[1] && c->operands[1] == body->args[0]);
    return uses_args && body->ops[1]->operands.size() == 1 && body->ops[1]->operands[0] == c->results[0];
  }
  // The row statistic `stat` (one value per row) broadcast along the row: broadcast_in_dim over the leading
  // dimensions, or, as jax spells keepdims, a reshape to [..., 1] broadcast over all dimensions. Returns the
  // operation that made the statistic, or null.
  Op* row_broadcast_source(Value* v, Block* b, int rank) {
    Op* bc = def_in(v, b, "broadcast_in_dim");
    if (!bc || uses[v] != 1 || bc->results[0]->type.rank() != rank) return nullptr;
    auto dims = attr_i64s(bc->attr("broadcast_dimensions"));
    Value* src = bc->operands[0];
    if (src->type.rank() == rank - 1 && (int)dims.size() == rank - 1) {
      for (int k = 0; k < rank - 1; k++) if (dims[k] != k) return nullptr;
      return src->def && src->def->parent == b ? src->def : nullptr;
    }
    if (src->type.rank() == rank && (int)dims.size() == rank && src->type.dims[rank - 1] == 1) {
      for (int k = 0; k < rank; k++) if (dims[k] != k) return nullptr;
      Op* rs = def_in(src, b, "reshape");
      if (!rs || uses[src] != 1 || rs->operands[0]->type.rank() != rank - 1) return nullptr;
      for (int k = 0; k < rank - 1; k++) if (rs->operands[0]->type.dims[k] != src->type.dims[k]) return nullptr;
      Value* inner = rs->operands[0];
      drop_too.push_back(rs);
      return inner->def && inner->def->parent == b ? inner->def : nullptr;
    }
    return nullptr;
  }
  std::vector<Op*> drop_too;               // reshapes between a statistic and its broadcast, dropped with the softmax
  // [G,] rows x cols operands contracted as dims say: batch = leading dimension (or none), contraction lc / rc
  static bool dot_form(Op* d, int lc, int rc) {
    if (d->operands.size() != 2 || d->results.size() != 1 || !d->has("dot_dimension_numbers")) return false;
    const int rank = d->operands[0]->type.rank();
    if (!(rank == 2 || rank == 3) || d->operands[1]->type.rank() != rank || d->results[0]->type.rank() != rank) return false;
    auto f = attr_struct(d->attr("dot_dimension_numbers"));
    const auto lb = f["lhs_batching_dimensions"], rb = f["rhs_batching_dimensions"];
    const auto lcd = f["lhs_contracting_dimensions"], rcd = f["rhs_contracting_dimensions"];
    if (rank == 2 ? !(lb.empty() && rb.empty()) : !(lb == std::vector<int64_t>{0} && rb == std::vector<int64_t>{0})) return false;
    return lcd == std::vector<int64_t>{(int64_t)(rank - 2 + lc)} && rcd == std::vector<int64_t>{(int64_t)(rank - 2 + rc)};
  }

  bool try_fuse(Block* b, Op* pv) {
    // ---- from the second product backwards through the softmax
    if (!dot_form(pv, 1, 0)) return false;
    Value* pin = pv->operands[0];
    Value* V = pv->operands[1];
    const int rank = pin->type.rank();
    Op* cvt = def_in(pin, b, "convert");
    Value* P = cvt ? cvt->operands[0] : pin;
    if (cvt && uses[pin] != 1) return false;
    Op* div = def_in(P, b, "divide");
    if (!div || uses[P] != 1 || P->type.dt != DT::F32) return false;
    Value* e = div->operands[0];
    drop_too.clear();
    Op* bs = def_in(div->operands[1], b, "broadcast_in_dim");
    Op* sum = row_broadcast_source(div->operands[1], b, rank);
    if (!bs || !sum || sum->short_name() != "reduce" || uses[sum->results[0]] != 1 || !last_dim_reduce(sum, "add") || sum->operands[0] != e || !splat_is(sum->operands[1], 0.0)) return false;
    Op* ex = def_in(e, b, "exponential");
    if (!ex || uses[e] != 2) return false;
    Op* sub = def_in(ex->operands[0], b, "subtract");
    if (!sub || uses[sub->results[0]] != 1) return false;
    Value* Sp = sub->operands[0];
    Op* bm = def_in(sub->operands[1], b, "broadcast_in_dim");
    Op* mx = row_broadcast_source(sub->operands[1], b, rank);
    if (!bm || !mx || mx->short_name() != "reduce" || uses[mx->results[0]] != 1 || !last_dim_reduce(mx, "maximum") || mx->operands[0] != Sp ||
        !splat_is(mx->operands[1], -std::numeric_limits<double>::infinity()))
      return false;
    if (uses[Sp] != 2 || Sp->type.dt != DT::F32 || Sp->type.dims != P->type.dims) return false;
    // ---- the pointwise part between the first product and the softmax
    std::set<Op*> seen, dots;
    std::vector<Op*> stack;
    if (Sp->def && Sp->def->parent == b) stack.push_back(Sp->def);
    while (!stack.empty()) {
      Op* o = stack.back();
      stack.pop_back();
      if (!seen.insert(o).second) continue;
      if (o->short_name() == "dot_general") { dots.insert(o); continue; }
      if (!is_elementwise_op(o->short_name()) || o->results.size() != 1) continue;
      for (Value* x : o->operands) if (x->def && x->def->parent == b) stack.push_back(x->def);
    }
    if (dots.size() != 1) return false;
    Op* qk = *dots.begin();
    if (!dot_form(qk, 1, 1)) return false;
    Value *Q = qk->operands[0], *K = qk->operands[1], *S = qk->results[0];
    if (uses[S] != 1 || S->type.dims != Sp->type.dims) return false;
    const DT dt = Q->type.dt;
    if (!(dt == DT::BF16 || dt == DT::F16) || K->type.dt != dt || V->type.dt != dt || pin->type.dt != dt) return false;
    if (!(S->type.dt == dt || S->type.dt == DT::F32)) return false;
    const DT odt = pv->results[0]->type.dt;
    if (!(odt == dt || odt == DT::F32)) return false;
    const int64_t M = Q->type.dims[rank - 2], D = Q->type.dims[rank - 1], T = K->type.dims[rank - 2], N = V->type.dims[rank - 1];
    const int64_t G = rank == 3 ? Q->type.dims[0] : 1;
    if (M < 1 || M > 8 || D % 8 || N % 8 || D < 8 || N < 8 || D > 256 || N > 256 || T < 1 || T >= (1 << 24) || G < 1 || G > 65535) return false;
    if (V->type.dims[rank - 2] != T || K->type.dims[rank - 1] != D) return false;
    if (rank == 3 && (K->type.dims[0] != G || V->type.dims[0] != G)) return false;
    // the operations that depend on S, in block order; nothing outside them may read their results
    std::set<Op*> moved;
    std::function<bool(Op*)> depends = [&](Op* o) -> bool {
      if (o == qk) return true;
      if (!seen.count(o) || o->short_name() == "dot_general" || !is_elementwise_op(o->short_name())) return false;
      bool any = false;
      for (Value* x : o->operands) if (x->def && x->def->parent == b && depends(x->def)) any = true;
      if (any) moved.insert(o);
      return any;
    };
    if (!Sp->def || !depends(Sp->def)) return false;
    for (Op* o : moved) {
      if (o->results[0] == Sp) continue;
      int inside = 0;
      for (Op* u : moved) for (Value* x : u->operands) if (x == o->results[0]) inside++;
      if (inside != uses[o->results[0]]) return false;
    }
    // operand subtrees of pointwise and duplicable operations that only the moved operations read move along, so
    // that the mask of a step is computed inside the kernel instead of by a launch of its own
    bool grew = true;
    while (grew) {
      grew = false;
      for (Op* o : std::vector<Op*>(moved.begin(), moved.end()))
        for (Value* x : o->operands) {
          Op* d = x->def;
          if (!d || d->parent != b || moved.count(d) || d == qk || d->results.size() != 1) continue;
          const std::string sh = d->short_name();
          if (!(is_elementwise_op(sh) || sh == "constant" || sh == "iota" || sh == "broadcast_in_dim")) continue;
          int inside = 0;
          for (Op* u : moved) for (Value* y : u->operands) if (y == x) inside++;
          if (inside != uses[x]) continue;
          moved.insert(d);
          grew = true;
        }
    }
    // ---- build the fused operation in place of the second product
    auto fused = std::make_unique<Op>();
    fused->name = "b200.decode_attention";
    fused->operands = {Q, K, V};
    fused->parent = b;
    fused->attrs["label"] = "\"attention M=" + std::to_string(M) + " T=" + std::to_string(T) + " D=" + std::to_string(D) + " N=" + std::to_string(N) + "\"";
    Value* out = pv->results[0];
    out->def = fused.get();
    out->def_index = 0;
    fused->results.push_back(out);
    auto body = std::make_unique<Block>();
    body->parent_op = fused.get();
    Value* sarg = m.new_value(S->type, "%scores");
    sarg->owner = body.get();
    sarg->arg_index = 0;
    body->args.push_back(sarg);
    std::set<Op*> gone = {qk, pv, div, bs, sum, ex, sub, bm, mx};
    if (cvt) gone.insert(cvt);
    for (Op* o : drop_too) gone.insert(o);
    std::vector<std::unique_ptr<Op>> kept;
    std::unique_ptr<Op> fused_holder = std::move(fused);
    for (auto& up : b->ops) {
      Op* o = up.get();
      if (o == pv) {
        Op* f = fused_holder.get();
        // finish the region before the operation takes the product's place
        auto ret = std::make_unique<Op>();
        ret->name = "stablehlo.return";
        ret->operands = {Sp};
        ret->parent = body.get();
        body->ops.push_back(std::move(ret));
        f->regions.push_back(std::move(body));
        kept.push_back(std::move(fused_holder));
        continue;
      }
      if (moved.count(o)) {
        for (auto& x : o->operands) if (x == S) x = sarg;
        o->parent = body.get();
        body->ops.push_back(std::move(up));
        continue;
      }
      if (gone.count(o)) {
        // reduce initial values and the like stay where they are; dead code elimination drops what nothing reads
        for (Value* r : o->results) if (r->def == o) r->def = nullptr;
        continue;
      }
      kept.push_back(std::move(up));
    }
    b->ops = std::move(kept);
    uses.clear();
    Block* top = b;
    while (top->parent_op && top->parent_op->parent) top = top->parent_op->parent;
    count(top);
    return true;
  }
};

// ---------------------------------------------------------------------------
// op classification
// ---------------------------------------------------------------------------
enum class Cat { ELEMENTWISE, DUP, INDEXING, REDUCE, DOT, CONV, SCATTER, WINDOW, SORT, RNG, LINALG, ATTENTION, WHILE, CASE, ALL_REDUCE, ALL_GATHER, RETURN, TOKEN, PARTITION_ID, UNSUPPORTED };

Cat categorize(Op* op) {
  const std::string sh = op->short_name();
  if (sh == "return") return Cat::RETURN;
  if (op->name == "b200.decode_attention") return Cat::ATTENTION;
  if (op->name.rfind("stablehlo.", 0) != 0 && op->name.rfind("chlo.", 0) != 0 && op->name.rfind("mhlo.", 0) != 0)
    return Cat::UNSUPPORTED;
  if (is_elementwise_op(sh)) return Cat::ELEMENTWISE;
  if (sh == "constant" || sh == "iota" || sh == "broadcast_in_dim") return Cat::DUP;
  if (sh == "reshape" || sh == "transpose" || sh == "reverse" || sh == "slice" || sh == "pad" || sh == "concatenate" ||
      sh == "dynamic_slice" || sh == "dynamic_update_slice" || sh == "gather")
    return Cat::INDEXING;
  if (sh == "reduce") return Cat::REDUCE;
  if (sh == "dot_general") return Cat::DOT;
  if (sh == "convolution") return Cat::CONV;
  if (sh == "scatter") return Cat::SCATTER;
  if (sh == "reduce_window" || sh == "select_and_scatter") return Cat::WINDOW;
  if (sh == "sort") return Cat::SORT;
  if (sh == "rng_bit_generator") return Cat::RNG;
  if (sh == "cholesky" || sh == "triangular_solve") return Cat::LINALG;
  if (sh == "while") return Cat::WHILE;
  if (sh == "case") return Cat::CASE;
  if (sh == "all_reduce") return Cat::ALL_REDUCE;
  if (sh == "all_gather") return Cat::ALL_GATHER;
  if (sh == "create_token" || sh == "after_all") return Cat::TOKEN;
  if (sh == "partition_id" || sh == "replica_id") return Cat::PARTITION_ID;
  return Cat::UNSUPPORTED;
}

void collect_unsupported(Block* b, std::set<std::string>& out, bool in_combiner) {
  for (auto& op : b->ops) {
    Cat c = categorize(op.get());
    if (c == Cat::UNSUPPORTED) out.insert(op->name);
    bool comb = c == Cat::REDUCE || c == Cat::SCATTER || c == Cat::WINDOW || c == Cat::SORT || c == Cat::ALL_REDUCE || c == Cat::ALL_GATHER;
    for (auto& r : op->regions) collect_unsupported(r.get(), out, comb);
  }
}

// ---------------------------------------------------------------------------
// planning
// ---------------------------------------------------------------------------
struct Group {
  int id = 0;
  bool is_reduce = false;
  std::set<Op*> members;            // non-duplicable ops evaluated inside the kernel (roots included)
  std::vector<Op*> roots;           // ops whose results are written to memory
  std::set<Op*> identity;           // members evaluated at the root's own index
  int max_pos = -1;
};

struct Unit {
  enum Kind { GROUP, OP, CONST_MAT } kind = OP;
  Group* group = nullptr;
  Op* op = nullptr;
  int prio = 0;
};

struct Planner {
  CompiledProgram& prog;
  const CompileOptions& opts;
  Module& mod;
  std::map<Value*, int> slot_of;
  std::map<std::string, int> kernel_cache;
  std::vector<std::string> kernel_text;       // un-named source of every generated kernel, by kernel id
  std::deque<Value> synth_values;
  std::ostringstream dump;
  int next_group_id = 0;

  Planner(CompiledProgram& p, const CompileOptions& o, Module& m) : prog(p), opts(o), mod(m) {}

  int new_slot(Slot::Kind kind, const TensorType& t, int arena) {
    Slot s;
    s.kind = kind;
    s.type = t;
    s.bytes = std::max<size_t>(t.bytes(), 1);
    s.arena = arena;
    prog.slots.push_back(s);
    return (int)prog.slots.size() - 1;
  }
  int const_slot(const TensorType& t, std::vector<uint8_t> bytes) {
    int s = new_slot(Slot::CONST, t, 0);
    prog.slots[s].index = (int)prog.consts.size();
    prog.slots[s].bytes = std::max<size_t>(bytes.size(), 1);
    prog.consts.push_back({std::move(bytes)});
    return s;
  }
  int table_slot(const void* data, size_t bytes) {
    TensorType t;
    t.dt = DT::U8;
    t.dims = {(int64_t)bytes};
    std::vector<uint8_t> v((const uint8_t*)data, (const uint8_t*)data + bytes);
    return const_slot(t, std::move(v));
  }
  Value* synth(const TensorType& t) {
    synth_values.emplace_back();
    Value* v = &synth_values.back();
    v->id = 1000000 + (int)synth_values.size();
    v->type = t;
    return v;
  }
  // `stem` names the kernel family in profiler listings ("fused", "reduce"); identical bodies share one kernel
  int add_kernel(const std::string& body_without_name, const char* stem) {
    auto it = kernel_cache.find(body_without_name);
    if (it != kernel_cache.end()) return it->second;
    int id = (int)prog.kernels.size();
    KernelSource ks;
    ks.name = std::string(stem) + "_" + std::to_string(id);
    std::string body = body_without_name;
    for (auto p = body.find("@NAME@"); p != std::string::npos; p = body.find("@NAME@", p)) body.replace(p, 6, ks.name);
    // every generated kernel can be launched with programmatic stream serialization: it lets the next kernel be
    // scheduled, then waits for everything in front of it before it touches memory
    {
      const size_t sig = body.find("__global__");
      const size_t open = sig == std::string::npos ? std::string::npos : body.find(") {\n", sig);
      if (open != std::string::npos) body.insert(open + 4, "  pdl_prologue();\n");
    }
    ks.body = body;
    prog.kernels.push_back(ks);
    kernel_cache[body_without_name] = id;
    kernel_text.push_back(body_without_name);
    return id;
  }

  // ---- per-block planning -------------------------------------------------
  struct BlockState {
    Block* block;
    int arena;
    std::vector<Op*> ops;
    std::map<Value*, std::vector<Op*>> users;       // users in this block (nested uses lifted to the region owner)
    std::set<Value*> returned;
    std::map<Op*, std::vector<Group*>> group_of;   // a cheap op may be evaluated in several kernels
    std::deque<Group> groups;
    std::set<Op*> dup_materialize;
  };

  static void lift_uses(Block* inner, Op* owner, Block* home, BlockState& st) {
    for (auto& op : inner->ops) {
      for (auto* o : op->operands) {
        // defined in `home` (op result or block argument)?
        bool in_home = (o->def && o->def->parent == home) || (!o->def && o->owner == home);
        if (in_home) st.users[o].push_back(owner);
      }
      for (auto& r : op->regions) lift_uses(r.get(), owner, home, st);
    }
  }

  bool is_dup(Op* op) { return categorize(op) == Cat::DUP; }
  bool fusable(Op* op) {
    Cat c = categorize(op);
    return c == Cat::ELEMENTWISE || c == Cat::INDEXING;
  }

  // May the value produced by `p` be computed inside the kernel of user `u`?
  bool can_fuse_into(Op* p, Value* pv, Op* u) {
    Cat cu = categorize(u);
    if (cu == Cat::ELEMENTWISE) return true;
    if (cu == Cat::INDEXING) {
      std::string sh = u->short_name();
      if (sh == "gather") return u->operands[0] != pv;       // table stays in memory; indices may be computed
      return true;
    }
    if (cu == Cat::REDUCE) {
      size_t n = u->operands.size() / 2;
      for (size_t k = n; k < u->operands.size(); k++)
        if (u->operands[k] == pv) return false;             // init values are read from memory
      return true;
    }
    return false;
  }

  // Would the kernel of group `g` have to run after any of the start ops / start groups have run?
  // Def-use edges are followed at the granularity of kernels: an op that is consumed inside a group makes
  // every output of that group "later"; a cheap op shared by several groups is no edge between them.
  bool reaches(const std::vector<Op*>& start_ops, const std::vector<Group*>& start_groups, Group* g, BlockState& st) {
    std::set<Op*> seen;
    std::set<Group*> seen_groups;
    std::vector<Op*> work;
    auto expand_group = [&](Group* h) {
      if (h == g || !seen_groups.insert(h).second) return;
      for (Op* r : h->roots)
        for (auto* res : r->results)
          for (auto* u : st.users[res]) work.push_back(u);
    };
    for (Group* h : start_groups) expand_group(h);
    for (Op* o : start_ops) work.push_back(o);
    while (!work.empty()) {
      Op* o = work.back();
      work.pop_back();
      if (!seen.insert(o).second) continue;
      if (g->members.count(o)) return true;          // reached through a def-use edge: g consumes a later value
      auto git = st.group_of.find(o);
      if (git != st.group_of.end()) {
        for (Group* h : git->second) expand_group(h);
        continue;
      }
      if (o->pos > g->max_pos) continue;
      for (auto* r : o->results)
        for (auto* u : st.users[r]) work.push_back(u);
    }
    return false;
  }

  static bool cheap_to_duplicate(Op* op) {
    if (categorize(op) != Cat::ELEMENTWISE) return false;
    static const std::set<std::string> cheap = {"add", "subtract", "multiply", "maximum", "minimum", "negate", "abs",
                                                "compare", "select", "convert", "and", "or", "xor", "not", "clamp", "sign"};
    return cheap.count(op->short_name()) != 0;
  }

  bool identity_in(Group* g, Op* op, BlockState& st) {
    Value* v = op->results[0];
    for (auto* u : st.users[v])
      if (g->identity.count(u) && categorize(u) == Cat::ELEMENTWISE && u->results[0]->type.dims == v->type.dims)
        return true;
    return false;
  }

  void build_groups(BlockState& st) {
    for (int i = (int)st.ops.size() - 1; i >= 0; i--) {
      Op* op = st.ops[i];
      Cat cat = categorize(op);
      if (cat == Cat::REDUCE) {
        st.groups.emplace_back();
        Group* g = &st.groups.back();
        g->id = next_group_id++;
        g->is_reduce = true;
        g->members.insert(op);
        g->roots.push_back(op);
        g->max_pos = op->pos;
        st.group_of[op].push_back(g);
        continue;
      }
      if (cat == Cat::DUP) {
        bool needs = st.returned.count(op->results[0]) != 0;
        for (auto* u : st.users[op->results[0]]) {
          Cat cu = categorize(u);
          bool inl = cu == Cat::ELEMENTWISE || cu == Cat::INDEXING || cu == Cat::DUP ||
                     (cu == Cat::REDUCE && can_fuse_into(op, op->results[0], u));
          if (cu == Cat::INDEXING && u->short_name() == "gather" && u->operands[0] == op->results[0]) inl = false;
          if (!inl) needs = true;
        }
        if (op->short_name() == "constant") {
          DenseValue dv = attr_dense(op->attr("value"));
          if (!dv.splat && dv.type.numel() > 0) needs = true;    // dense data always lives in memory
        }
        if (needs) st.dup_materialize.insert(op);
        continue;
      }
      if (!fusable(op)) continue;
      Value* v = op->results[0];
      std::vector<Group*> gs;          // groups of users that can evaluate this op inline
      std::vector<Op*> ext;            // users that need the value in memory
      bool returned = st.returned.count(v) != 0;
      for (auto* u : st.users[v]) {
        auto it = st.group_of.find(u);
        if (opts.fuse && it != st.group_of.end() && can_fuse_into(op, v, u)) {
          for (auto* g : it->second)
            if (std::find(gs.begin(), gs.end(), g) == gs.end()) gs.push_back(g);
        } else ext.push_back(u);
      }
      auto join = [&](Group* g, bool as_root) {
        g->members.insert(op);
        st.group_of[op].push_back(g);
        if (as_root) { g->roots.push_back(op); g->identity.insert(op); }
        else if (identity_in(g, op, st)) g->identity.insert(op);
      };
      if (ext.empty() && !returned && gs.size() == 1) { join(gs[0], false); continue; }
      if (ext.empty() && !returned && gs.size() > 1 && cheap_to_duplicate(op)) {
        bool small = true;
        for (auto* g : gs) small &= g->members.size() < 48;
        // a chain of duplicated operations (the residual stream of a deep network: x4 = x3 + o3 = x2 + o2 + o3 ...)
        // would be re-evaluated from ever more inputs by every later kernel: after four links the value is written
        int depth = 1;
        for (auto* u : st.users[v]) {
          auto du = dup_depth.find(u);
          if (du != dup_depth.end()) depth = std::max(depth, du->second + 1);
        }
        if (depth > 8) small = false;
        if (small) {
          dup_depth[op] = depth;
          for (auto* g : gs) join(g, false);
          continue;
        }
      }
      // written to memory: as an extra output of a consumer kernel when it shares that kernel's index space
      std::sort(gs.begin(), gs.end(), [](Group* a, Group* b) { return a->max_pos < b->max_pos; });
      bool placed = false;
      for (auto* g : gs) {
        if (g->is_reduce || !identity_in(g, op, st)) continue;
        // consumers that will read the value from memory: non-fusable users, and every other group
        // holding one of its users
        std::vector<Op*> others = ext;
        std::vector<Group*> other_groups;
        for (auto* u : st.users[v]) {
          auto it = st.group_of.find(u);
          if (it == st.group_of.end()) continue;
          for (Group* h : it->second)
            if (h != g && std::find(other_groups.begin(), other_groups.end(), h) == other_groups.end())
              other_groups.push_back(h);
        }
        if (reaches(others, other_groups, g, st)) continue;
        join(g, true);
        placed = true;
        break;
      }
      if (placed) continue;
      st.groups.emplace_back();
      Group* g = &st.groups.back();
      g->id = next_group_id++;
      g->members.insert(op);
      g->roots.push_back(op);
      g->identity.insert(op);
      g->max_pos = op->pos;
      st.group_of[op].push_back(g);
    }
  }

  // Reductions over the same index space that read common inputs (batch-norm statistics sum x / sum x^2, the
  // two or three sums of its gradient) become one kernel with several accumulators, so the inputs are read
  // once. Legal when neither kernel has to run after the other (checked at kernel granularity both ways).
  void merge_sibling_reductions(BlockState& st) {
    auto inputs_of = [&](Group* g) {
      std::set<Value*> in;
      for (Op* m : g->members)
        for (Value* o : m->operands)
          if (!(o->def && g->members.count(o->def))) in.insert(o);
      return in;
    };
    std::vector<Group*> reds;
    for (auto& g : st.groups)
      if (g.is_reduce && g.roots.size() == 1 && !g.members.empty()) reds.push_back(&g);
    std::sort(reds.begin(), reds.end(), [](Group* a, Group* b) { return a->max_pos < b->max_pos; });
    for (size_t i = 0; i < reds.size(); i++) {
      Group* a = reds[i];
      if (a->members.empty()) continue;
      for (size_t j = i + 1; j < reds.size(); j++) {
        Group* b = reds[j];
        if (b->members.empty() || b->max_pos - a->max_pos > 4096) continue;
        Op *ra = a->roots[0], *rb = b->roots[0];
        if (ra->operands[0]->type.dims != rb->operands[0]->type.dims) continue;
        if (attr_i64s(ra->attr("dimensions")) != attr_i64s(rb->attr("dimensions"))) continue;
        if (a->roots.size() + b->roots.size() > 4 || a->members.size() + b->members.size() > 96) continue;
        auto ia = inputs_of(a), ib = inputs_of(b);
        bool shared = false;
        for (Value* v : ia)
          if (ib.count(v) && v->type.numel() * 4 >= ra->operands[0]->type.numel()) { shared = true; break; }
        if (!shared) continue;
        if (reaches({}, {a}, b, st) || reaches({}, {b}, a, st)) continue;
        // b joins a
        for (Op* m : b->members) {
          a->members.insert(m);
          auto& gs = st.group_of[m];
          gs.erase(std::remove(gs.begin(), gs.end(), b), gs.end());
          if (std::find(gs.begin(), gs.end(), a) == gs.end()) gs.push_back(a);
        }
        for (Op* r : b->roots) a->roots.push_back(r);
        a->max_pos = std::max(a->max_pos, b->max_pos);
        b->members.clear();
        b->roots.clear();
      }
    }
  }

  // ---- kernel generation -----------------------------------------------------
  struct Launch {
    int kernel;
    unsigned grid[3], block[3];
    std::vector<Value*> outs, ins;
  };

  std::string idx_type_for(const std::vector<Value*>& vals, int64_t extra = 0) {
    int64_t mx = extra;
    for (auto* v : vals) mx = std::max<int64_t>(mx, v->type.numel());
    return mx >= (1LL << 31) - 1024 ? "i64" : "int";
  }

  std::string store_expr(DT d, const std::string& e) {
    if (d == DT::BF16) return "f_to_bf16(" + e + ")";
    if (d == DT::F16) return "f_to_f16(" + e + ")";
    if (d == DT::PRED) return "(u8)(" + e + ")";
    return e;
  }

  std::string signature(const std::vector<Value*>& outs, const std::vector<Value*>& ins) {
    std::string s;
    for (size_t k = 0; k < outs.size(); k++)
      s += std::string(k ? ", " : "") + s_type(outs[k]->type.dt) + "* __restrict__ out" + std::to_string(k);
    for (size_t k = 0; k < ins.size(); k++)
      s += std::string((k || !outs.empty()) ? ", " : "") + "const " + s_type(ins[k]->type.dt) + "* __restrict__ in" +
           std::to_string(k);
    return s;
  }

  // replaces `from` by `to` where `from` does not continue an identifier; true when anything was replaced
  static bool replace_word(std::string& str, const std::string& from, const std::string& to) {
    size_t pos = 0;
    bool any = false;
    while ((pos = str.find(from, pos)) != std::string::npos) {
      if (pos > 0 && (isalnum((unsigned char)str[pos - 1]) || str[pos - 1] == '_')) { pos += from.size(); continue; }
      str.replace(pos, from.size(), to);
      pos += to.size();
      any = true;
    }
    return any;
  }

  // moves W elements of `es` bytes between a thread's array `arr` and `ptr + base` in the widest aligned pieces
  static std::string wide_move(const std::string& arr, const std::string& ptr, int W, int es, bool is_load, int indent = 2) {
    std::ostringstream o;
    const int bytes = W * es;
    const char* piece = bytes >= 16 ? "uint4" : (bytes == 8 ? "uint2" : "unsigned int");
    const int pb = bytes >= 16 ? 16 : bytes;
    for (int q = 0; q < bytes / pb; q++) {
      const std::string mem = "reinterpret_cast<" + std::string(is_load ? "const " : "") + piece + "*>(" + ptr + " + base)[" + std::to_string(q) + "]";
      const std::string loc = "reinterpret_cast<" + std::string(is_load ? "" : "const ") + piece + "*>(" + arr + ")[" + std::to_string(q) + "]";
      o << std::string(indent, ' ') << (is_load ? loc + " = " + mem : mem + " = " + loc) << ";\n";
    }
    return o.str();
  }

  static constexpr int kEPT = 4;       // elements per thread of a pointwise kernel
  static constexpr int kThreads = 256;

  Launch gen_pointwise(Group* g, BlockState& st) {
    std::vector<Value*> outs;
    for (auto* r : g->roots) outs.push_back(r->results[0]);
    const TensorType& rt = outs[0]->type;
    for (auto* o : outs)
      if (o->type.dims != rt.dims) throw CompileError("internal: fused outputs of different shapes");
    int64_t n = rt.numel();
    Emitter em;
    em.is_internal = [&](Op* o) { return g->members.count(o) || (is_dup(o) && !st.dup_materialize.count(o) && !slot_of.count(o->results[0])); };
    std::vector<Value*> all;
    for (auto* m : g->members) {
      all.push_back(m->results[0]);
      for (auto* o : m->operands) all.push_back(o);
    }
    em.idx_t = idx_type_for(all, n + kThreads * 8);
    Ctx root;
    root.shape = rt.dims;
    root.lin = "lin";
    em.ensure_idx(root);
    std::vector<std::string> vals;
    for (auto* o : outs) vals.push_back(em.emit(o, root));
    for (size_t k = 0; k < outs.size(); k++)
      em.line("out" + std::to_string(k) + "[lin] = " + store_expr(outs[k]->type.dt, vals[k]) + ";");
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << signature(outs, em.inputs)
        << ") {\n";
    // Wide accesses: a thread takes W consecutive elements (8 when a 2-byte type is among the outputs and the element
    // count allows it, else 4). Inputs read at the kernel's own linear index (same-shaped tensors) are fetched with
    // 16-byte loads (one for 8 two-byte or 4 four-byte elements, two for 8 four-byte ones), the outputs leave the
    // same way. Other operands (broadcast vectors, gathers) keep their scalar loads.
    auto esize = [](DT d) -> int {
      switch (d) {
        case DT::F32: case DT::I32: case DT::U32: return 4;
        case DT::BF16: case DT::F16: case DT::I16: case DT::U16: return 2;
        case DT::PRED: case DT::I8: case DT::U8: return 1;
        default: return 0;
      }
    };
    bool two_byte_out = false, wide_ok = n >= 4096;
    for (auto* o : outs) {
      wide_ok = wide_ok && esize(o->type.dt) != 0;
      two_byte_out = two_byte_out || esize(o->type.dt) == 2;
    }
    const int W = (two_byte_out && n % 8 == 0) ? 8 : 4;
    for (auto* o : outs) wide_ok = wide_ok && (W * esize(o->type.dt)) % 4 == 0;
    const bool vec4 = wide_ok && n % W == 0 && !getenv("B200_NO_WIDE_POINTWISE");
    Launch L;
    if (vec4) {
      std::string body = em.str();
      std::ostringstream loads, stores;
      for (size_t k = 0; k < em.inputs.size(); k++) {
        Value* in = em.inputs[k];
        const int es = esize(in->type.dt);
        if (es == 0 || (W * es) % 4 != 0 || in->type.numel() != n) continue;
        const std::string nm = "in" + std::to_string(k);
        if (!replace_word(body, nm + "[lin]", "v" + nm + "[e]")) continue;
        loads << "  __align__(16) " << s_type(in->type.dt) << " v" << nm << "[" << W << "];\n" << wide_move("v" + nm, nm, W, es, true);
      }
      for (size_t k = 0; k < outs.size(); k++) {
        const std::string nm = "out" + std::to_string(k);
        replace_word(body, nm + "[lin]", "v" + nm + "[e]");
        loads << "  __align__(16) " << s_type(outs[k]->type.dt) << " v" << nm << "[" << W << "];\n";
        stores << wide_move("v" + nm, nm, W, esize(outs[k]->type.dt), false);
      }
      src << "  const " << em.idx_t << " base = ((" << em.idx_t << ")blockIdx.x * " << kThreads << " + threadIdx.x) * " << W << ";\n";
      src << "  if (base >= (" << em.idx_t << ")" << n << "LL) return;\n";
      src << loads.str();
      src << "  #pragma unroll\n  for (int e = 0; e < " << W << "; ++e) {\n";
      src << "    const " << em.idx_t << " lin = base + e;\n";
      src << body;
      src << "  }\n" << stores.str() << "}\n";
      L.kernel = add_kernel(src.str(), "fused");
      int64_t blocks = std::max<int64_t>(1, (n / W + kThreads - 1) / kThreads);
      L.grid[0] = (unsigned)blocks; L.grid[1] = L.grid[2] = 1;
    } else {
      src << "  #pragma unroll\n  for (int e = 0; e < " << kEPT << "; ++e) {\n";
      src << "    const " << em.idx_t << " lin = ((" << em.idx_t << ")blockIdx.x * " << kEPT << " + e) * " << kThreads
          << " + threadIdx.x;\n";
      src << "    if (lin >= (" << em.idx_t << ")" << n << "LL) break;\n";
      src << em.str();
      src << "  }\n}\n";
      L.kernel = add_kernel(src.str(), "fused");
      int64_t blocks = std::max<int64_t>(1, (n + (int64_t)kThreads * kEPT - 1) / ((int64_t)kThreads * kEPT));
      L.grid[0] = (unsigned)blocks; L.grid[1] = L.grid[2] = 1;
    }
    L.block[0] = kThreads; L.block[1] = L.block[2] = 1;
    L.outs = outs;
    L.ins = em.inputs;
    return L;
  }

  // ---- window operations (src/pjrt_plugin/ops/reduction.cc:165-626 of the reference) ---------------------------------
  // Geometry of a window operation: per dimension the window size, stride, padding in front, base (input) dilation and
  // window dilation. `padding` is dense<...> : tensor<R x 2 x i64> (possibly a splat), the rest array<i64: ...>.
  struct WindowGeom { std::vector<int64_t> win, stride, pad_lo, bdil, wdil; };
  WindowGeom window_geometry(Op* op, int rank) {
    WindowGeom g;
    auto list = [&](const char* name, int64_t dflt) {
      std::vector<int64_t> v = op->has(name) ? attr_i64s(op->attr(name)) : std::vector<int64_t>();
      if (v.empty()) v.assign(rank, dflt);
      if ((int)v.size() != rank) throw CompileError(op->name + ": " + name + " must have one entry per dimension");
      return v;
    };
    g.win = list("window_dimensions", 1);
    g.stride = list("window_strides", 1);
    g.bdil = list("base_dilations", 1);
    g.wdil = list("window_dilations", 1);
    g.pad_lo.assign(rank, 0);
    if (op->has("padding")) {
      DenseValue d = attr_dense(op->attr("padding"));
      if (d.type.numel() != 2 * rank || dt_size(d.type.dt) != 8) throw CompileError(op->name + ": padding must be a [rank, 2] i64 tensor");
      for (int k = 0; k < rank; k++) memcpy(&g.pad_lo[k], d.data.data() + 16 * k, 8);
    }
    for (int k = 0; k < rank; k++)
      if (g.win[k] < 1 || g.stride[k] < 1 || g.bdil[k] < 1 || g.wdil[k] < 1) throw CompileError(op->name + ": window sizes, strides and dilations must be positive");
    return g;
  }

  // the value of element `at` of input `v` of a hand-assembled kernel (storage type -> compute type)
  static std::string load_expr(Value* v, const std::string& name, const std::string& at) {
    std::string e = name + "[" + at + "]";
    if (v->type.dt == DT::BF16) return "bf16_to_f(" + e + ")";
    if (v->type.dt == DT::F16) return "f16_to_f(" + e + ")";
    if (v->type.dt == DT::PRED) return "(" + e + " != 0)";
    return e;
  }

  // stablehlo.reduce_window (pooling, cumulative sums): one thread per output element walks its window; positions
  // in the padding, or between the elements of a dilated input, contribute the init value. The body may be any
  // reduction computation (it is emitted as it stands), with several inputs reduced together.
  Launch gen_reduce_window(Op* op, BlockState& st) {
    const size_t n = op->operands.size() / 2;
    if (n < 1 || op->operands.size() != 2 * n || op->results.size() != n || op->regions.size() != 1)
      throw CompileError("stablehlo.reduce_window: malformed operands");
    const TensorType& it = op->operands[0]->type;
    const TensorType& ot = op->results[0]->type;
    const int R = it.rank();
    if (ot.rank() != R) throw CompileError("stablehlo.reduce_window: result rank differs from the input's");
    WindowGeom g = window_geometry(op, R);
    std::vector<Value*> ins;
    for (size_t k = 0; k < 2 * n; k++) {
      if (!slot_of.count(op->operands[k])) throw CompileError("internal: operand of reduce_window has no storage");
      ins.push_back(op->operands[k]);
    }
    std::vector<Value*> outs(op->results.begin(), op->results.end());
    Emitter em;
    em.is_internal = [](Op*) { return false; };
    em.idx_t = idx_type_for(ins, ot.numel() + kThreads);
    em.indent_ = 2;
    Ctx root;
    root.shape = ot.dims;
    root.lin = "lin";
    em.ensure_idx(root);
    const std::string I = em.idx_t;
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << signature(outs, ins) << ") {\n";
    src << "  const " << I << " lin = (" << I << ")blockIdx.x * " << kThreads << " + threadIdx.x;\n";
    src << "  if (lin >= (" << I << ")" << ot.numel() << "LL) return;\n";
    src << em.str();
    for (size_t k = 0; k < n; k++)
      src << "  const " << c_type(ins[n + k]->type.dt) << " init" << k << " = " << load_expr(ins[n + k], "in" + std::to_string(n + k), "0") << ";\n"
          << "  " << c_type(outs[k]->type.dt) << " acc" << k << " = init" << k << ";\n";
    std::vector<int64_t> istr(R, 1);
    for (int d = R - 2; d >= 0; d--) istr[d] = istr[d + 1] * it.dims[d + 1];
    for (int d = 0; d < R; d++) {
      const std::string w = "w" + std::to_string(d);
      src << "  for (int " << w << " = 0; " << w << " < " << g.win[d] << "; ++" << w << ") {\n";
      // position in the dilated, padded input, then the input element it falls on (if any)
      src << "  const long long p" << d << " = (long long)" << (root.idx[d] == "0" ? std::string("0") : root.idx[d]) << " * " << g.stride[d] << " + " << w << " * "
          << g.wdil[d] << " - " << g.pad_lo[d] << ";\n";
      src << "  const bool ok" << d << " = " << (d ? "ok" + std::to_string(d - 1) + " && " : "") << "p" << d << " >= 0 && p" << d << " % " << g.bdil[d]
          << " == 0 && p" << d << " / " << g.bdil[d] << " < " << it.dims[d] << ";\n";
    }
    {
      std::string at;
      for (int d = 0; d < R; d++) at += (d ? " + " : "") + std::string("(p") + std::to_string(d) + " / " + std::to_string(g.bdil[d]) + ") * " + std::to_string(istr[d]) + "LL";
      if (R == 0) at = "0";
      const std::string okl = R ? "ok" + std::to_string(R - 1) : "true";
      Emitter be;
      be.idx_t = I;
      be.name_prefix = "b";
      be.indent_ = 2;
      be.round_small_floats = true;
      std::vector<std::string> args;
      for (size_t k = 0; k < n; k++) args.push_back("acc" + std::to_string(k));
      for (size_t k = 0; k < n; k++) {
        be.line(std::string("const ") + c_type(ins[k]->type.dt) + " val" + std::to_string(k) + " = " + okl + " ? " +
                load_expr(ins[k], "in" + std::to_string(k), "(" + I + ")(" + okl + " ? " + at + " : 0)") + " : init" + std::to_string(k) + ";");
        args.push_back("val" + std::to_string(k));
      }
      auto res = be.emit_scalar_region(op->regions[0].get(), args);
      for (size_t k = 0; k < n; k++) be.line("acc" + std::to_string(k) + " = " + res[k] + ";");
      src << be.str();
    }
    for (int d = 0; d < R; d++) src << "  }\n";
    for (size_t k = 0; k < n; k++) src << "  out" << k << "[lin] = " << store_expr(outs[k]->type.dt, "acc" + std::to_string(k)) << ";\n";
    src << "}\n";
    Launch L;
    L.kernel = add_kernel(src.str(), "window");
    L.grid[0] = (unsigned)std::max<int64_t>(1, (ot.numel() + kThreads - 1) / kThreads); L.grid[1] = L.grid[2] = 1;
    L.block[0] = kThreads; L.block[1] = L.block[2] = 1;
    L.outs = outs;
    L.ins = ins;
    return L;
  }

  // stablehlo.select_and_scatter (the gradient of max / min pooling): in gather form, so that it is deterministic. One
  // thread per operand element visits the windows that cover it in row-major order of the windows; for each it scans
  // the window's in-bounds elements in row-major order with the select computation (the current choice stays while
  // select(current, candidate) holds, so ties go to the first element for GE / LE and to the last for GT / LT; padding is
  // never selected, as in the reference) and, when the chosen element is its own, folds the window's source value into its
  // result with the scatter computation, starting from the init value.
  Launch gen_select_and_scatter(Op* op, BlockState& st) {
    if (op->operands.size() != 3 || op->results.size() != 1 || op->regions.size() != 2)
      throw CompileError("stablehlo.select_and_scatter: malformed operands");
    Value *operand = op->operands[0], *source = op->operands[1], *init = op->operands[2], *out = op->results[0];
    const TensorType& ot = operand->type;
    const TensorType& stt = source->type;
    const int R = ot.rank();
    if (stt.rank() != R) throw CompileError("stablehlo.select_and_scatter: source rank differs from the operand's");
    WindowGeom g = window_geometry(op, R);
    for (int d = 0; d < R; d++)
      if (g.bdil[d] != 1 || g.wdil[d] != 1) throw CompileError("stablehlo.select_and_scatter has no dilations");
    for (Value* v : {operand, source, init})
      if (!slot_of.count(v)) throw CompileError("internal: operand of select_and_scatter has no storage");
    std::vector<Value*> ins = {operand, source, init}, outs = {out};
    Emitter em;
    em.is_internal = [](Op*) { return false; };
    em.idx_t = idx_type_for(ins, ot.numel() + kThreads);
    em.indent_ = 2;
    Ctx root;
    root.shape = ot.dims;
    root.lin = "lin";
    em.ensure_idx(root);
    const std::string I = em.idx_t;
    std::vector<int64_t> ostr(R, 1), sstr(R, 1);
    for (int d = R - 2; d >= 0; d--) { ostr[d] = ostr[d + 1] * ot.dims[d + 1]; sstr[d] = sstr[d + 1] * stt.dims[d + 1]; }
    const char* ct = c_type(ot.dt);
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << signature(outs, ins) << ") {\n";
    src << "  const " << I << " lin = (" << I << ")blockIdx.x * " << kThreads << " + threadIdx.x;\n";
    src << "  if (lin >= (" << I << ")" << ot.numel() << "LL) return;\n";
    src << em.str();
    src << "  " << ct << " acc = " << load_expr(init, "in2", "0") << ";\n";
    // windows that cover this element: s * stride <= i + pad < s * stride + win
    for (int d = 0; d < R; d++) {
      const std::string i = root.idx[d] == "0" ? "0" : root.idx[d];
      src << "  const long long q" << d << " = (long long)" << i << " + " << g.pad_lo[d] << ";\n";
      src << "  const long long slo" << d << " = q" << d << " - " << (g.win[d] - 1) << " <= 0 ? 0 : (q" << d << " - " << (g.win[d] - 1) << " + " << (g.stride[d] - 1)
          << ") / " << g.stride[d] << ";\n";
      src << "  const long long shi" << d << " = q" << d << " < 0 ? -1 : (q" << d << " / " << g.stride[d] << " < " << stt.dims[d] << " ? q" << d << " / " << g.stride[d]
          << " : " << (stt.dims[d] - 1) << ");\n";
    }
    for (int d = 0; d < R; d++) src << "  for (long long s" << d << " = slo" << d << "; s" << d << " <= shi" << d << "; ++s" << d << ") {\n";
    src << "  bool have = false;\n  " << ct << " cur = acc;\n  long long cur_at = -1;\n";
    for (int d = 0; d < R; d++) {
      src << "  for (int w" << d << " = 0; w" << d << " < " << g.win[d] << "; ++w" << d << ") {\n";
      src << "  const long long p" << d << " = s" << d << " * " << g.stride[d] << " + w" << d << " - " << g.pad_lo[d] << ";\n";
      src << "  const bool ok" << d << " = " << (d ? "ok" + std::to_string(d - 1) + " && " : "") << "p" << d << " >= 0 && p" << d << " < " << ot.dims[d] << ";\n";
    }
    {
      std::string at;
      for (int d = 0; d < R; d++) at += (d ? " + " : "") + std::string("p") + std::to_string(d) + " * " + std::to_string(ostr[d]) + "LL";
      if (R == 0) at = "0";
      const std::string okl = R ? "ok" + std::to_string(R - 1) : "true";
      Emitter se;
      se.idx_t = I;
      se.name_prefix = "s";
      se.indent_ = 2;
      se.line("if (" + okl + ") {");
      se.line("const long long at = " + at + ";");
      se.line(std::string("const ") + ct + " cand = " + load_expr(operand, "in0", "at") + ";");
      se.line("bool keep = false;");
      se.line("if (have) {");
      auto res = se.emit_scalar_region(op->regions[0].get(), {"cur", "cand"});
      se.line("keep = " + res[0] + ";");
      se.line("}");
      se.line("if (!keep) { cur = cand; cur_at = at; have = true; }");
      se.line("}");
      src << se.str();
    }
    for (int d = 0; d < R; d++) src << "  }\n";
    {
      std::string sat;
      for (int d = 0; d < R; d++) sat += (d ? " + " : "") + std::string("s") + std::to_string(d) + " * " + std::to_string(sstr[d]) + "LL";
      if (R == 0) sat = "0";
      Emitter ce;
      ce.idx_t = I;
      ce.name_prefix = "c";
      ce.indent_ = 2;
      ce.line("if (have && cur_at == (long long)lin) {");
      ce.line(std::string("const ") + c_type(source->type.dt) + " sv = " + load_expr(source, "in1", sat) + ";");
      auto res = ce.emit_scalar_region(op->regions[1].get(), {"acc", "sv"});
      ce.line("acc = " + res[0] + ";");
      ce.line("}");
      src << ce.str();
    }
    for (int d = 0; d < R; d++) src << "  }\n";
    src << "  out0[lin] = " << store_expr(out->type.dt, "acc") << ";\n}\n";
    Launch L;
    L.kernel = add_kernel(src.str(), "window");
    L.grid[0] = (unsigned)std::max<int64_t>(1, (ot.numel() + kThreads - 1) / kThreads); L.grid[1] = L.grid[2] = 1;
    L.block[0] = kThreads; L.block[1] = L.block[2] = 1;
    L.outs = outs;
    L.ins = ins;
    return L;
  }

  // stablehlo.sort (src/pjrt_plugin/ops/sort_fft_complex.cc:135-250 of the reference, which recognises ascending and
  // descending comparators; here the comparator region is compiled as it stands). A stable merge sort over a
  // permutation: a block sorts a tile of up to kSortTile elements of one row in shared memory, starting from runs of
  // one element and doubling; every element finds its place in the merged run by a binary search of the sibling run
  // (elements of the left run go before equal elements of the right run, which is what makes the sort stable for any
  // strict weak order). Rows longer than a tile continue with one launch per doubling over a permutation in global
  // memory; the last pass of either kind writes the sorted operands. All operands move together.
  static constexpr int kSortTile = 1024;
  void lower_sort(Op* op, Plan& plan, BlockState& st) {
    const size_t k = op->operands.size();
    if (k < 1 || op->results.size() != k || op->regions.size() != 1 || op->regions[0]->args.size() != 2 * k)
      throw CompileError("stablehlo.sort: malformed operands or comparator");
    const TensorType& t0 = op->operands[0]->type;
    const int R = t0.rank();
    int64_t dim = op->has("dimension") ? attr_int(op->attr("dimension")) : R - 1;
    if (dim < 0) dim += R;
    if (R == 0 || dim < 0 || dim >= R) throw CompileError("stablehlo.sort: dimension out of range");
    int64_t smem = 0;
    for (size_t q = 0; q < k; q++) {
      if (op->operands[q]->type.dims != t0.dims || !(op->results[q]->type == op->operands[q]->type))
        throw CompileError("stablehlo.sort: operands and results must share one shape");
      if (!slot_of.count(op->operands[q])) throw CompileError("internal: operand of sort has no storage");
      smem += dt_size(op->operands[q]->type.dt);
    }
    std::vector<Value*> ins(op->operands.begin(), op->operands.end()), outs(op->results.begin(), op->results.end());
    for (auto* o : outs) ensure_slot(o, st);
    const int64_t N = t0.dims[dim], numel = t0.numel();
    if (numel == 0) return;
    int64_t inner = 1;
    for (int d = (int)dim + 1; d < R; d++) inner *= t0.dims[d];
    const int64_t rows = numel / N;
    if (N >= (1LL << 30)) throw CompileError("stablehlo.sort: more than 2^30 elements along the sorted dimension");
    if (smem * kSortTile > 36 * 1024) throw CompileError("stablehlo.sort: operands of more than 36 bytes per element together are not supported");
    const int64_t tiles = (N + kSortTile - 1) / kSortTile;
    if (rows * tiles >= (1LL << 31)) throw CompileError("stablehlo.sort: too many rows");
    const bool one_tile = tiles == 1;

    // shared pieces of source text
    auto comparator = [&](Emitter& e) {
      // bool before(a0, b0, a1, b1, ...): the comparator region on compute types
      std::string sig;
      std::vector<std::string> args;
      for (size_t q = 0; q < k; q++) {
        const std::string ct = c_type(ins[q]->type.dt);
        sig += (q ? ", " : "") + ct + " a" + std::to_string(q) + ", " + ct + " b" + std::to_string(q);
        args.push_back("a" + std::to_string(q));
        args.push_back("b" + std::to_string(q));
      }
      e.line("auto before = [&](" + sig + ") -> bool {");
      auto res = e.emit_scalar_region(op->regions[0].get(), args);
      if (res.size() != 1) throw CompileError("stablehlo.sort: the comparator must return one value");
      e.line("return " + res[0] + ";");
      e.line("};");
    };
    auto row_base = [&](std::ostringstream& src) {
      src << "  const long long base = (row / " << inner << "LL) * " << (N * inner) << "LL + row % " << inner << "LL;\n";
    };
    auto call_before = [&](const std::string& x, const std::string& y) {
      std::string c = "before(";
      for (size_t q = 0; q < k; q++) c += (q ? ", " : "") + x + std::to_string(q) + ", " + y + std::to_string(q);
      return c + ")";
    };

    int perm[2] = {-1, -1};
    if (!one_tile) {
      TensorType pt;
      pt.dt = DT::I32;
      pt.dims = {numel};
      perm[0] = new_slot(Slot::TEMP, pt, st.arena);
      perm[1] = new_slot(Slot::TEMP, pt, st.arena);
    }
    // ---- tile kernel
    {
      std::ostringstream src;
      src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(";
      if (one_tile) src << signature(outs, ins);
      else src << "int* __restrict__ perm_out, " << signature({}, ins);
      src << ") {\n";
      src << "  __shared__ int sp[2][" << kSortTile << "];\n";
      for (size_t q = 0; q < k; q++) src << "  __shared__ " << s_type(ins[q]->type.dt) << " sv" << q << "[" << kSortTile << "];\n";
      src << "  const long long row = (long long)blockIdx.x / " << tiles << ";\n";
      src << "  const int t0 = (int)((long long)blockIdx.x % " << tiles << ") * " << kSortTile << ";\n";
      src << "  const int cnt = " << N << " - t0 < " << kSortTile << " ? " << N << " - t0 : " << kSortTile << ";\n";
      row_base(src);
      src << "  for (int i = threadIdx.x; i < cnt; i += " << kThreads << ") {\n    sp[0][i] = i;\n";
      for (size_t q = 0; q < k; q++) src << "    sv" << q << "[i] = in" << q << "[base + (long long)(t0 + i) * " << inner << "LL];\n";
      src << "  }\n  __syncthreads();\n";
      Emitter ce;
      ce.idx_t = "int";
      ce.name_prefix = "c";
      ce.indent_ = 2;
      comparator(ce);
      src << ce.str();
      src << "  int cur = 0;\n";
      src << "  for (int w = 1; w < cnt; w <<= 1) {\n";
      src << "    for (int i = threadIdx.x; i < cnt; i += " << kThreads << ") {\n";
      src << "      const int run = i / (2 * w) * (2 * w);\n";
      src << "      const bool right = i - run >= w;\n";
      src << "      const int me = sp[cur][i];\n";
      for (size_t q = 0; q < k; q++) src << "      const " << c_type(ins[q]->type.dt) << " a" << q << " = " << load_expr(ins[q], "sv" + std::to_string(q), "me") << ";\n";
      src << "      int lo = right ? run : run + w;\n";
      src << "      int hi = right ? run + w : run + 2 * w;\n";
      src << "      if (hi > cnt) hi = cnt;\n      if (lo > hi) lo = hi;\n";
      src << "      int l = lo, h = hi;\n";
      src << "      while (l < h) {\n        const int mid = (l + h) >> 1;\n        const int other = sp[cur][mid];\n";
      for (size_t q = 0; q < k; q++) src << "        const " << c_type(ins[q]->type.dt) << " b" << q << " = " << load_expr(ins[q], "sv" + std::to_string(q), "other") << ";\n";
      src << "        const bool goes_first = right ? !" << call_before("a", "b") << " : " << call_before("b", "a") << ";\n";
      src << "        if (goes_first) l = mid + 1; else h = mid;\n      }\n";
      src << "      sp[cur ^ 1][run + (right ? i - run - w : i - run) + (l - lo)] = me;\n";
      src << "    }\n    __syncthreads();\n    cur ^= 1;\n  }\n";
      src << "  for (int i = threadIdx.x; i < cnt; i += " << kThreads << ") {\n";
      if (one_tile) {
        for (size_t q = 0; q < k; q++) src << "    out" << q << "[base + (long long)(t0 + i) * " << inner << "LL] = sv" << q << "[sp[cur][i]];\n";
      } else {
        src << "    perm_out[row * " << N << "LL + t0 + i] = t0 + sp[cur][i];\n";
      }
      src << "  }\n}\n";
      Step s;
      s.kind = Step::KERNEL;
      s.kernel = add_kernel(src.str(), "sort_tile");
      s.label = "sort (tiles)";
      s.grid[0] = (unsigned)(rows * tiles); s.grid[1] = s.grid[2] = 1;
      s.block[0] = kThreads; s.block[1] = s.block[2] = 1;
      if (one_tile) { for (auto* o : outs) s.args.push_back(slot_of.at(o)); s.n_outs = (int)k; }
      else { s.args.push_back(perm[0]); s.n_outs = 1; }
      for (auto* i : ins) s.args.push_back(slot_of.at(i));
      plan.steps.push_back(std::move(s));
    }
    if (one_tile) return;
    // ---- merge passes: the width of the sorted runs comes from a constant, so that all passes but the last share a kernel
    int merge_kernel[2] = {-1, -1};          // [writes the operands]
    auto merge_source = [&](bool final_pass) {
      std::ostringstream src;
      src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(";
      if (final_pass) src << signature(outs, ins);
      else src << "int* __restrict__ perm_out, " << signature({}, ins);
      src << ", const int* __restrict__ perm_in, const int* __restrict__ width) {\n";
      src << "  const long long lin = (long long)blockIdx.x * " << kThreads << " + threadIdx.x;\n";
      src << "  if (lin >= " << numel << "LL) return;\n";
      src << "  const long long row = lin / " << N << "LL;\n  const long long i = lin % " << N << "LL;\n";
      row_base(src);
      src << "  const int* __restrict__ P = perm_in + row * " << N << "LL;\n";
      src << "  const long long w = width[0];\n";
      Emitter ce;
      ce.idx_t = "int";
      ce.name_prefix = "c";
      ce.indent_ = 2;
      comparator(ce);
      src << ce.str();
      src << "  const long long run = i / (2 * w) * (2 * w);\n";
      src << "  const bool right = i - run >= w;\n";
      src << "  const int me = P[i];\n";
      for (size_t q = 0; q < k; q++) src << "  const " << c_type(ins[q]->type.dt) << " a" << q << " = " << load_expr(ins[q], "in" + std::to_string(q), "base + (long long)me * " + std::to_string(inner) + "LL") << ";\n";
      src << "  long long lo = right ? run : run + w;\n";
      src << "  long long hi = right ? run + w : run + 2 * w;\n";
      src << "  if (hi > " << N << "LL) hi = " << N << "LL;\n  if (lo > hi) lo = hi;\n";
      src << "  long long l = lo, h = hi;\n";
      src << "  while (l < h) {\n    const long long mid = (l + h) >> 1;\n    const int other = P[mid];\n";
      for (size_t q = 0; q < k; q++) src << "    const " << c_type(ins[q]->type.dt) << " b" << q << " = " << load_expr(ins[q], "in" + std::to_string(q), "base + (long long)other * " + std::to_string(inner) + "LL") << ";\n";
      src << "    const bool goes_first = right ? !" << call_before("a", "b") << " : " << call_before("b", "a") << ";\n";
      src << "    if (goes_first) l = mid + 1; else h = mid;\n  }\n";
      src << "  const long long dest = run + (right ? i - run - w : i - run) + (l - lo);\n";
      if (final_pass) {
        for (size_t q = 0; q < k; q++) src << "  out" << q << "[base + dest * " << inner << "LL] = in" << q << "[base + (long long)me * " << inner << "LL];\n";
      } else {
        src << "  perm_out[row * " << N << "LL + dest] = me;\n";
      }
      src << "}\n";
      return src.str();
    };
    int from = 0;
    for (int64_t w = kSortTile; w < N; w <<= 1) {
      const bool final_pass = 2 * w >= N;
      int& kern = merge_kernel[final_pass ? 1 : 0];
      if (kern < 0) kern = add_kernel(merge_source(final_pass), final_pass ? "sort_merge_out" : "sort_merge");
      TensorType wt;
      wt.dt = DT::I32;
      std::vector<uint8_t> wb(4);
      const int32_t w32 = (int32_t)w;
      memcpy(wb.data(), &w32, 4);
      const int wslot = const_slot(wt, wb);
      Step s;
      s.kind = Step::KERNEL;
      s.kernel = kern;
      s.label = "sort (merge runs of " + std::to_string(w) + ")";
      s.grid[0] = (unsigned)((numel + kThreads - 1) / kThreads); s.grid[1] = s.grid[2] = 1;
      s.block[0] = kThreads; s.block[1] = s.block[2] = 1;
      if (final_pass) { for (auto* o : outs) s.args.push_back(slot_of.at(o)); s.n_outs = (int)k; }
      else { s.args.push_back(perm[from ^ 1]); s.n_outs = 1; }
      for (auto* i : ins) s.args.push_back(slot_of.at(i));
      s.args.push_back(perm[from]);
      s.args.push_back(wslot);
      plan.steps.push_back(std::move(s));
      from ^= 1;
    }
  }

  // stablehlo.rng_bit_generator (src/pjrt_plugin/ops/control_flow.cc:2301-2362 of the reference: bits from the
  // library's generator keyed by the first two state words, the counter in the state advanced by one per 16 bytes of
  // output; which algorithm the attribute names is not distinguished there, nor here). The state is 16 bytes (a 64-bit
  // key, then a 64-bit counter) or 24 bytes (the counter 128 bits wide). The output, read as bytes, is the start of the
  // Philox-4x32-10 stream of that key from that counter on: 16 bytes per counter value, words in little-endian order,
  // so that consecutive calls with the returned state continue the stream without overlap. One thread per counter value.
  void lower_rng_bit_generator(Op* op, Plan& plan, BlockState& st) {
    if (op->operands.size() != 1 || op->results.size() != 2) throw CompileError("stablehlo.rng_bit_generator: malformed operands");
    Value *state = op->operands[0], *out_state = op->results[0], *out = op->results[1];
    const size_t sbytes = state->type.bytes();
    if (!(sbytes == 16 || sbytes == 24) || !(state->type == out_state->type) || !(dt_is_unsigned(state->type.dt) || dt_is_signed(state->type.dt)))
      throw CompileError("stablehlo.rng_bit_generator: the state must be 16 or 24 bytes of integers, got " + state->type.str());
    if (!(dt_is_unsigned(out->type.dt) || dt_is_signed(out->type.dt)))
      throw CompileError("stablehlo.rng_bit_generator: the output must be of an integer type, got " + out->type.str());
    if (!slot_of.count(state)) throw CompileError("internal: state of rng_bit_generator has no storage");
    ensure_slot(out_state, st);
    ensure_slot(out, st);
    const long long bytes = (long long)out->type.numel() * dt_size(out->type.dt);
    const long long blocks = (bytes + 15) / 16;
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << s_type(state->type.dt) << "* __restrict__ out_state, "
        << s_type(out->type.dt) << "* __restrict__ out, const " << s_type(state->type.dt) << "* __restrict__ state) {\n";
    src << "  const u32* sw = (const u32*)state;\n";
    src << "  const u32 k0 = sw[0], k1 = sw[1];\n";
    src << "  const u64 lo64 = (u64)sw[2] | ((u64)sw[3] << 32);\n";
    src << "  const u64 hi64 = " << (sbytes == 24 ? "(u64)sw[4] | ((u64)sw[5] << 32)" : "0") << ";\n";
    src << "  const long long j = (long long)blockIdx.x * " << kThreads << " + threadIdx.x;\n";
    src << "  if (j == 0) {\n    u32* ow = (u32*)out_state;\n    const u64 lo = lo64 + " << blocks << "ULL;\n";
    src << "    ow[0] = k0; ow[1] = k1; ow[2] = (u32)lo; ow[3] = (u32)(lo >> 32);\n";
    if (sbytes == 24) src << "    const u64 hi = hi64 + (lo < lo64 ? 1ULL : 0ULL);\n    ow[4] = (u32)hi; ow[5] = (u32)(hi >> 32);\n";
    src << "  }\n";
    src << "  if (j >= " << blocks << "LL) return;\n";
    src << "  const u64 lo = lo64 + (u64)j;\n  const u64 hi = hi64 + (lo < lo64 ? 1ULL : 0ULL);\n";
    src << "  u32 r[4];\n  philox4x32_10((u32)lo, (u32)(lo >> 32), (u32)hi, (u32)(hi >> 32), k0, k1, r);\n";
    src << "  if ((j + 1) * 16 <= " << bytes << "LL) {\n    ((uint4*)out)[j] = make_uint4(r[0], r[1], r[2], r[3]);\n  } else {\n";
    src << "    for (int q = 0; q < (int)(" << bytes << "LL - j * 16); ++q) ((u8*)out)[j * 16 + q] = (u8)(r[q >> 2] >> (8 * (q & 3)));\n  }\n}\n";
    Step s;
    s.kind = Step::KERNEL;
    s.kernel = add_kernel(src.str(), "rng_bits");
    s.label = op->name;
    s.grid[0] = (unsigned)std::max<long long>(1, (blocks + kThreads - 1) / kThreads); s.grid[1] = s.grid[2] = 1;
    s.block[0] = kThreads; s.block[1] = s.block[2] = 1;
    s.args = {slot_of.at(out_state), slot_of.at(out), slot_of.at(state)};
    s.n_outs = 2;
    plan.steps.push_back(std::move(s));
  }

  // b200.decode_attention (DecodeAttentionFusion): attention of M <= 8 query rows per group over T cached positions in
  // one kernel. A block takes 32 positions of one group: it stages their K and V rows and the queries in shared
  // memory, its warps form the scores (rounded like the product they replace), the region's pointwise code (scale,
  // mask) runs on each score, a warp per query row takes the chunk's maximum and exponentials and multiplies them into
  // its part of the V rows. With more than one chunk, the chunk's unnormalised result, maximum and sum go to scratch,
  // and the last block of the group to arrive (a counter that it sets back to zero) rescales and adds the chunks in
  // chunk order and divides by the total. Unlike the chain it replaces, the probabilities are not rounded to 16 bits
  // on their way into the second product.
  void lower_decode_attention(Op* op, Plan& plan, BlockState& st) {
    Value *Q = op->operands[0], *K = op->operands[1], *V = op->operands[2], *out = op->results[0];
    Block* body = op->regions[0].get();
    Value* sarg = body->args[0];
    Value* Sp = body->ops.back()->operands[0];
    const int rank = Q->type.rank();
    const long long M = Q->type.dims[rank - 2], D = Q->type.dims[rank - 1], T = K->type.dims[rank - 2], N = V->type.dims[rank - 1];
    const long long G = rank == 3 ? Q->type.dims[0] : 1;
    const int TC = 32;
    const long long CH = (T + TC - 1) / TC, D8 = D / 8, N8 = N / 8, PS = N + 4;
    for (Value* v : {Q, K, V})
      if (!slot_of.count(v)) throw CompileError("internal: operand of decode_attention has no storage");
    ensure_slot(out, st);
    std::set<Op*> inside;
    for (auto& o : body->ops) inside.insert(o.get());
    Emitter em;
    em.is_internal = [&](Op* o) { return inside.count(o) || (is_dup(o) && !st.dup_materialize.count(o) && !slot_of.count(o->results[0])); };
    std::vector<Value*> all{Sp};
    for (auto& o : body->ops) for (Value* x : o->operands) all.push_back(x);
    em.idx_t = idx_type_for(all, G * M * T + 1024);
    em.indent_ = 6;
    em.bound[sarg] = "sval";
    Ctx root;
    root.shape = Sp->type.dims;
    root.lin = "lin";
    em.ensure_idx(root);
    const std::string rexpr = em.emit(Sp, root);
    for (Value* v : em.inputs)
      if (!slot_of.count(v)) throw CompileError("internal: value read by the attention region has no storage: " + v->name);
    const bool bf = Q->type.dt == DT::BF16;
    const std::string H2F = bf ? "bf16_to_f" : "f16_to_f";
    const std::string round_s = sarg->type.dt == DT::F32 ? "mine" : (bf ? "rbf16(mine)" : "rf16(mine)");
    const std::string I = em.idx_t;
    auto unpack = [&](const std::string& vec, const std::string& arr) {
      std::string o;
      const char* comp[4] = {"x", "y", "z", "w"};
      for (int q = 0; q < 4; q++) {
        o += "        " + arr + "[" + std::to_string(2 * q) + "] = " + H2F + "((u16)(" + vec + "." + comp[q] + " & 0xFFFFu));\n";
        o += "        " + arr + "[" + std::to_string(2 * q + 1) + "] = " + H2F + "((u16)(" + vec + "." + comp[q] + " >> 16));\n";
      }
      return o;
    };
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(256) @NAME@(" << s_type(out->type.dt) << "* __restrict__ out0, float* __restrict__ part, "
        << "int* __restrict__ cnt, const u16* __restrict__ qp, const u16* __restrict__ kp, const u16* __restrict__ vp";
    if (!em.inputs.empty()) src << ", " << signature({}, em.inputs);
    src << ") {\n";
    src << "  __shared__ __align__(16) u16 ks[" << TC * D << "];\n  __shared__ __align__(16) u16 vs[" << TC * N << "];\n";
    src << "  __shared__ __align__(16) float qs[" << M * D << "];\n  __shared__ float sc[" << M * TC << "];\n  __shared__ int last_flag;\n";
    src << "  const int c = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;\n";
    src << "  const int t0 = c * " << TC << ";\n  const int nt = " << T << " - t0 < " << TC << " ? " << T << " - t0 : " << TC << ";\n";
    src << "  const float NEG_INF = __uint_as_float(0xFF800000u);\n";
    src << "  {\n    const uint4* ksrc = (const uint4*)(kp + ((long long)g * " << T << " + t0) * " << D << ");\n";
    src << "    for (int i = tid; i < nt * " << D8 << "; i += 256) ((uint4*)ks)[i] = ksrc[i];\n";
    src << "    const uint4* vsrc = (const uint4*)(vp + ((long long)g * " << T << " + t0) * " << N << ");\n";
    src << "    for (int i = tid; i < nt * " << N8 << "; i += 256) ((uint4*)vs)[i] = vsrc[i];\n";
    src << "    for (int i = tid; i < " << M * D << "; i += 256) qs[i] = " << H2F << "(qp[(long long)g * " << M * D << " + i]);\n  }\n";
    src << "  __syncthreads();\n";
    // scores
    src << "  for (int tl = warp; tl < nt; tl += 8) {\n    float acc[" << M << "];\n";
    src << "#pragma unroll\n    for (int m = 0; m < " << M << "; ++m) acc[m] = 0.f;\n";
    src << "    for (int p = lane; p < " << D8 << "; p += 32) {\n      const uint4 kk = ((const uint4*)ks)[tl * " << D8 << " + p];\n      float kf[8];\n";
    src << unpack("kk", "kf");
    src << "#pragma unroll\n      for (int m = 0; m < " << M << "; ++m) {\n        const float4 qa = *(const float4*)(qs + m * " << D << " + p * 8), qb = *(const float4*)(qs + m * " << D << " + p * 8 + 4);\n";
    src << "        acc[m] = fmaf(kf[0], qa.x, acc[m]); acc[m] = fmaf(kf[1], qa.y, acc[m]); acc[m] = fmaf(kf[2], qa.z, acc[m]); acc[m] = fmaf(kf[3], qa.w, acc[m]);\n";
    src << "        acc[m] = fmaf(kf[4], qb.x, acc[m]); acc[m] = fmaf(kf[5], qb.y, acc[m]); acc[m] = fmaf(kf[6], qb.z, acc[m]); acc[m] = fmaf(kf[7], qb.w, acc[m]);\n      }\n    }\n";
    src << "    float mine = 0.f;\n#pragma unroll\n    for (int m = 0; m < " << M << "; ++m) {\n      float r = acc[m];\n";
    src << "#pragma unroll\n      for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xFFFFFFFFu, r, o);\n      if (lane == m) mine = r;\n    }\n";
    src << "    if (lane < " << M << ") sc[lane * " << TC << " + tl] = mine;\n  }\n  __syncthreads();\n";
    // the pointwise part on every score of the chunk at once (its loads, a mask for instance, go out together)
    src << "  for (int i = tid; i < " << M * TC << "; i += 256) {\n    const int mrow = i / " << TC << ", tl = i % " << TC << ";\n    if (tl < nt) {\n";
    src << "      const float mine = sc[i];\n      const float sval = " << round_s << ";\n";
    src << "      const " << I << " lin = ((" << I << ")g * " << M << " + mrow) * " << T << " + t0 + tl;\n";
    src << em.str();
    src << "      sc[i] = " << rexpr << ";\n    }\n  }\n  __syncthreads();\n";
    // softmax of the chunk and the second product, a warp per query row
    src << "  if (warp < " << M << ") {\n    const int mrow = warp;\n    float mx = NEG_INF;\n";
    src << "    for (int tl = lane; tl < nt; tl += 32) mx = fmaxf(mx, sc[mrow * " << TC << " + tl]);\n";
    src << "#pragma unroll\n    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));\n";
    src << "    const float mref = mx == NEG_INF ? 0.f : mx;\n    float sum = 0.f;\n";
    src << "    for (int tl = lane; tl < nt; tl += 32) { const float pz = expf(sc[mrow * " << TC << " + tl] - mref); sc[mrow * " << TC << " + tl] = pz; sum += pz; }\n";
    src << "#pragma unroll\n    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);\n    __syncwarp();\n";
    src << "    for (int p = lane; p < " << N8 << "; p += 32) {\n      float o8[8];\n#pragma unroll\n      for (int e = 0; e < 8; ++e) o8[e] = 0.f;\n";
    src << "      for (int tl = 0; tl < nt; ++tl) {\n        const float pz = sc[mrow * " << TC << " + tl];\n        const uint4 vv = ((const uint4*)vs)[tl * " << N8 << " + p];\n        float vf[8];\n";
    src << unpack("vv", "vf");
    src << "#pragma unroll\n        for (int e = 0; e < 8; ++e) o8[e] = fmaf(pz, vf[e], o8[e]);\n      }\n";
    if (CH == 1) {
      src << "#pragma unroll\n      for (int e = 0; e < 8; ++e) out0[((long long)g * " << M << " + mrow) * " << N << " + p * 8 + e] = " << store_expr(out->type.dt, "(o8[e] / sum)") << ";\n";
      src << "    }\n  }\n}\n";
    } else {
      src << "      float* dst = part + (((long long)g * " << CH << " + c) * " << M << " + mrow) * " << PS << " + p * 8;\n";
      src << "      *(float4*)dst = make_float4(o8[0], o8[1], o8[2], o8[3]);\n      *(float4*)(dst + 4) = make_float4(o8[4], o8[5], o8[6], o8[7]);\n    }\n";
      src << "    if (lane == 0) {\n      float* dst = part + (((long long)g * " << CH << " + c) * " << M << " + mrow) * " << PS << " + " << N << ";\n      dst[0] = mx;\n      dst[1] = sum;\n    }\n  }\n";
      src << "  __threadfence();\n  __syncthreads();\n";
      src << "  if (tid == 0) last_flag = atomicAdd(cnt + g, 1) == " << (CH - 1) << ";\n  __syncthreads();\n  if (!last_flag) return;\n  __threadfence();\n";
      src << "  if (warp < " << M << ") {\n    const int mrow = warp;\n    const float* base = part + ((long long)g * " << CH * M << " + mrow) * " << PS << ";\n";
      // lanes take the chunks' maxima and sums side by side: the row's maximum, then every chunk's weight and the total
      src << "    float gm = NEG_INF;\n    for (int cc = lane; cc < " << CH << "; cc += 32) gm = fmaxf(gm, __ldcg(base + (long long)cc * " << M * PS << " + " << N << "));\n";
      src << "#pragma unroll\n    for (int o = 16; o > 0; o >>= 1) gm = fmaxf(gm, __shfl_xor_sync(0xFFFFFFFFu, gm, o));\n";
      src << "    float den = 0.f, wl = 0.f;\n    for (int cc = lane; cc < " << CH << "; cc += 32) {\n      const float mc = __ldcg(base + (long long)cc * " << M * PS << " + " << N << ");\n";
      src << "      wl = mc == NEG_INF ? 0.f : expf(mc - gm);\n      den += wl * __ldcg(base + (long long)cc * " << M * PS << " + " << (N + 1) << ");\n    }\n";
      src << "#pragma unroll\n    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xFFFFFFFFu, den, o);\n";
      src << "    for (int p = lane; p < " << ((N8 + 31) / 32 * 32) << "; p += 32) {\n      const bool mine = p < " << N8 << ";\n      float o8[8];\n#pragma unroll\n      for (int e = 0; e < 8; ++e) o8[e] = 0.f;\n";
      src << "#pragma unroll " << std::min<long long>(CH, 10) << "\n      for (int cc = 0; cc < " << CH << "; ++cc) {\n        const float* row = base + (long long)cc * " << M * PS << ";\n";
      if (CH <= 32) src << "        const float w = __shfl_sync(0xFFFFFFFFu, wl, cc);\n";
      else src << "        const float mc = __ldcg(row + " << N << ");\n        const float w = mc == NEG_INF ? 0.f : expf(mc - gm);\n";
      src << "        if (!mine) continue;\n";
      src << "        const float4 a = __ldcg((const float4*)(row + p * 8)), b4 = __ldcg((const float4*)(row + p * 8 + 4));\n";
      src << "        o8[0] = fmaf(w, a.x, o8[0]); o8[1] = fmaf(w, a.y, o8[1]); o8[2] = fmaf(w, a.z, o8[2]); o8[3] = fmaf(w, a.w, o8[3]);\n";
      src << "        o8[4] = fmaf(w, b4.x, o8[4]); o8[5] = fmaf(w, b4.y, o8[5]); o8[6] = fmaf(w, b4.z, o8[6]); o8[7] = fmaf(w, b4.w, o8[7]);\n      }\n";
      src << "      if (!mine) continue;\n";
      src << "#pragma unroll\n      for (int e = 0; e < 8; ++e) out0[((long long)g * " << M << " + mrow) * " << N << " + p * 8 + e] = " << store_expr(out->type.dt, "(o8[e] / den)") << ";\n";
      src << "    }\n  }\n  if (tid == 0) cnt[g] = 0;\n}\n";
    }
    Step s;
    s.kind = Step::KERNEL;
    s.kernel = add_kernel(src.str(), "attention");
    s.label = op->has("label") ? attr_str(op->attr("label")) : op->name;
    s.grid[0] = (unsigned)CH; s.grid[1] = (unsigned)G; s.grid[2] = 1;
    s.block[0] = 256; s.block[1] = s.block[2] = 1;
    TensorType pt;
    pt.dt = DT::F32;
    pt.dims = {std::max<long long>(1, CH > 1 ? G * CH * M * PS : 1)};
    std::vector<int> zeros((size_t)G, 0);
    s.args = {slot_of.at(out), new_slot(Slot::TEMP, pt, st.arena), table_slot(zeros.data(), zeros.size() * sizeof(int)), slot_of.at(Q), slot_of.at(K), slot_of.at(V)};
    for (Value* v : em.inputs) s.args.push_back(slot_of.at(v));
    s.n_outs = 3;
    plan.steps.push_back(std::move(s));
  }

  // stablehlo.cholesky (src/pjrt_plugin/ops/linalg.cc:553-570 of the reference hands it to LAPACK on the host). One
  // block per matrix factors it in place in the result, column by column: the square root of the pivot, the column
  // scaled by it, then the trailing triangle updated with the column's outer product; every element is written by one
  // thread per step, so the result does not depend on scheduling. Only the named triangle of the input is read; the
  // other triangle of the result is zero. A matrix that is not positive definite gives NaN from its first bad pivot on.
  void lower_cholesky(Op* op, Plan& plan, BlockState& st) {
    if (op->operands.size() != 1 || op->results.size() != 1) throw CompileError("stablehlo.cholesky: malformed operands");
    Value *a = op->operands[0], *out = op->results[0];
    const int R = a->type.rank();
    if (R < 2 || a->type.dims[R - 1] != a->type.dims[R - 2] || !(a->type == out->type))
      throw CompileError("stablehlo.cholesky: the operand must be a batch of square matrices, got " + a->type.str());
    if (!(a->type.dt == DT::F32 || a->type.dt == DT::F64)) throw CompileError("stablehlo.cholesky: element type " + a->type.str() + " is not supported (f32, f64)");
    if (!slot_of.count(a)) throw CompileError("internal: operand of cholesky has no storage");
    ensure_slot(out, st);
    const int64_t n = a->type.dims[R - 1], batch = n ? a->type.numel() / (n * n) : 0;
    if (batch == 0 || n == 0) return;
    if (n > 46340 || batch >= (1LL << 31)) throw CompileError("stablehlo.cholesky: matrix or batch too large");
    const bool lower = !op->has("lower") || attr_bool(op->attr("lower"));
    const std::string T = c_type(a->type.dt);
    const std::string at = lower ? "(i) * N + (j)" : "(j) * N + (i)";        // element (i, j) of the lower factor
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << signature({out}, {a}) << ") {\n";
    src << "#define AT(i, j) (" << at << ")\n";
    src << "  const int N = " << n << ";\n";
    src << "  " << T << "* o = out0 + (long long)blockIdx.x * N * N;\n  const " << T << "* a = in0 + (long long)blockIdx.x * N * N;\n";
    src << "  for (int e = threadIdx.x; e < N * N; e += " << kThreads << ") { const int i = e / N, j = e % N; o[AT(i, j)] = i >= j ? a[AT(i, j)] : (" << T << ")0; }\n";
    src << "  __syncthreads();\n";
    src << "  for (int j = 0; j < N; ++j) {\n";
    src << "    if (threadIdx.x == 0) o[AT(j, j)] = op_sqrt(o[AT(j, j)]);\n    __syncthreads();\n";
    src << "    const " << T << " d = o[AT(j, j)];\n";
    src << "    for (int i = j + 1 + threadIdx.x; i < N; i += " << kThreads << ") o[AT(i, j)] = o[AT(i, j)] / d;\n    __syncthreads();\n";
    src << "    const int m = N - j - 1;\n";
    src << "    for (int e = threadIdx.x; e < m * m; e += " << kThreads << ") {\n      const int i = j + 1 + e / m, k = j + 1 + e % m;\n";
    src << "      if (k <= i) o[AT(i, k)] = o[AT(i, k)] - o[AT(i, j)] * o[AT(k, j)];\n    }\n    __syncthreads();\n  }\n";
    src << "#undef AT\n}\n";
    Step s;
    s.kind = Step::KERNEL;
    s.kernel = add_kernel(src.str(), "cholesky");
    s.label = op->name;
    s.grid[0] = (unsigned)batch; s.grid[1] = s.grid[2] = 1;
    s.block[0] = kThreads; s.block[1] = s.block[2] = 1;
    s.args = {slot_of.at(out), slot_of.at(a)};
    s.n_outs = 1;
    plan.steps.push_back(std::move(s));
  }

  // stablehlo.triangular_solve (src/pjrt_plugin/ops/linalg.cc:573-660 of the reference): op(A) X = B or X op(A) = B for a
  // batch of triangular A. One thread per right-hand-side vector (a column of B on the left side, a row on the right)
  // substitutes forwards or backwards through its matrix, reading its earlier unknowns back from the result. As in the
  // reference, a matrix with a zero on a diagonal that counts gives NaN for its whole solution.
  void lower_triangular_solve(Op* op, Plan& plan, BlockState& st) {
    if (op->operands.size() != 2 || op->results.size() != 1) throw CompileError("stablehlo.triangular_solve: malformed operands");
    Value *a = op->operands[0], *bv = op->operands[1], *out = op->results[0];
    const int R = a->type.rank();
    if (R < 2 || bv->type.rank() != R || a->type.dims[R - 1] != a->type.dims[R - 2] || !(bv->type == out->type) || a->type.dt != bv->type.dt)
      throw CompileError("stablehlo.triangular_solve: malformed operand types " + a->type.str() + ", " + bv->type.str());
    if (!(a->type.dt == DT::F32 || a->type.dt == DT::F64)) throw CompileError("stablehlo.triangular_solve: element type " + a->type.str() + " is not supported (f32, f64)");
    for (int d = 0; d < R - 2; d++) if (a->type.dims[d] != bv->type.dims[d]) throw CompileError("stablehlo.triangular_solve: batch dimensions differ");
    if (!slot_of.count(a) || !slot_of.count(bv)) throw CompileError("internal: operand of triangular_solve has no storage");
    ensure_slot(out, st);
    const bool left = !op->has("left_side") || attr_bool(op->attr("left_side"));
    const bool lower = !op->has("lower") || attr_bool(op->attr("lower"));
    const bool unit = op->has("unit_diagonal") && attr_bool(op->attr("unit_diagonal"));
    const std::string tr = op->has("transpose_a") ? attr_enum(op->attr("transpose_a")) : "NO_TRANSPOSE";
    const bool transposed = tr == "TRANSPOSE" || tr == "ADJOINT";
    const int64_t n = a->type.dims[R - 1], rows = bv->type.dims[R - 2], cols = bv->type.dims[R - 1];
    if ((left ? rows : cols) != n) throw CompileError("stablehlo.triangular_solve: B does not match A");
    const int64_t total = bv->type.numel();
    if (total == 0) return;
    const int64_t vecs_per = left ? cols : rows, batch = total / (rows * cols);
    const bool flip = transposed != !left;                 // the matrix the substitution walks is A transposed
    const bool fwd = lower != flip;                        // ... and it is lower triangular: substitute forwards
    const std::string T = c_type(a->type.dt);
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << signature({out}, {a, bv}) << ") {\n";
    src << "  const long long t = (long long)blockIdx.x * " << kThreads << " + threadIdx.x;\n";
    src << "  if (t >= " << batch * vecs_per << "LL) return;\n";
    src << "  const int N = " << n << ";\n";
    src << "  const long long g = t / " << vecs_per << "LL, v = t % " << vecs_per << "LL;\n";
    src << "  const " << T << "* A = in0 + g * N * N;\n";
    src << "#define M(i, j) A[" << (flip ? "(long long)(j) * N + (i)" : "(long long)(i) * N + (j)") << "]\n";
    src << "#define X(i) (g * " << rows * cols << "LL + " << (left ? "(long long)(i) * " + std::to_string(cols) + " + v" : "v * " + std::to_string(cols) + " + (i)") << ")\n";
    src << "  bool singular = false;\n";
    if (!unit) src << "  for (int i = 0; i < N; ++i) singular = singular || A[(long long)i * N + i] == (" << T << ")0;\n";
    src << "  for (int q = 0; q < N; ++q) {\n    const int i = " << (fwd ? "q" : "N - 1 - q") << ";\n";
    src << "    " << T << " acc = in1[X(i)];\n";
    src << "    for (int j = " << (fwd ? "0; j < i" : "i + 1; j < N") << "; ++j) acc = acc - M(i, j) * out0[X(j)];\n";
    src << "    out0[X(i)] = " << (unit ? "acc" : "acc / M(i, i)") << ";\n  }\n";
    src << "  if (singular) for (int i = 0; i < N; ++i) out0[X(i)] = (" << T << ")__uint_as_float(0x7FC00000u);\n";
    src << "#undef M\n#undef X\n}\n";
    Step s;
    s.kind = Step::KERNEL;
    s.kernel = add_kernel(src.str(), "triangular_solve");
    s.label = op->name;
    s.grid[0] = (unsigned)((batch * vecs_per + kThreads - 1) / kThreads); s.grid[1] = s.grid[2] = 1;
    s.block[0] = kThreads; s.block[1] = s.block[2] = 1;
    s.args = {slot_of.at(out), slot_of.at(a), slot_of.at(bv)};
    s.n_outs = 1;
    plan.steps.push_back(std::move(s));
  }

  // dynamic_update_slice of a loop-carried tensor written back to the same position of the loop state: the result
  // shares the state's memory and the kernel stores only the update window (one thread per update element)
  // instead of rewriting the whole tensor every iteration. Start indices are clamped as in the general form.
  Launch gen_window_update(Group* g, BlockState& st) {
    Op* d = g->roots[0];
    Value* out = d->results[0];
    Value* u = d->operands[1];
    const std::vector<int64_t>& od = out->type.dims;
    const int64_t n = u->type.numel();
    Emitter em;
    em.is_internal = [&](Op* o) {
      return (o != d && g->members.count(o)) || (is_dup(o) && !st.dup_materialize.count(o) && !slot_of.count(o->results[0]));
    };
    std::vector<Value*> all{out};
    for (auto* m : g->members) {
      all.push_back(m->results[0]);
      for (auto* o : m->operands) all.push_back(o);
    }
    em.idx_t = idx_type_for(all, n + kThreads * kEPT);
    Ctx uc;
    uc.shape = u->type.dims;
    uc.lin = "lin";
    em.ensure_idx(uc);
    std::string dst;
    int64_t stride = 1;
    std::vector<int64_t> strides(od.size());
    for (size_t i = od.size(); i-- > 0;) { strides[i] = stride; stride *= od[i]; }
    for (size_t i = 0; i < od.size(); i++) {
      Ctx sc;
      sc.lin = "0";
      std::string sv = em.emit(d->operands[2 + i], sc);
      std::string nv = em.fresh("s");
      em.line("const " + em.idx_t + " " + nv + " = (" + em.idx_t + ")min(max((i64)" + sv + ", (i64)0), (i64)" +
              std::to_string(od[i] - u->type.dims[i]) + ");");
      dst += std::string(i ? " + " : "") + "(" + nv + " + " + uc.idx[i] + ") * (" + em.idx_t + ")" + std::to_string(strides[i]) + "LL";
    }
    std::string val = em.emit(u, uc);
    em.line("out0[" + dst + "] = " + store_expr(out->type.dt, val) + ";");
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << signature({out}, em.inputs) << ") {\n";
    src << "  #pragma unroll\n  for (int e = 0; e < " << kEPT << "; ++e) {\n";
    src << "    const " << em.idx_t << " lin = ((" << em.idx_t << ")blockIdx.x * " << kEPT << " + e) * " << kThreads
        << " + threadIdx.x;\n";
    src << "    if (lin >= (" << em.idx_t << ")" << n << "LL) break;\n";
    src << em.str();
    src << "  }\n}\n";
    Launch L;
    L.kernel = add_kernel(src.str(), "fused");
    int64_t blocks = std::max<int64_t>(1, (n + (int64_t)kThreads * kEPT - 1) / ((int64_t)kThreads * kEPT));
    L.grid[0] = (unsigned)blocks; L.grid[1] = L.grid[2] = 1;
    L.block[0] = kThreads; L.block[1] = L.block[2] = 1;
    L.outs = {out};
    L.ins = em.inputs;
    return L;
  }

  // A reduction kernel over `in_shape` along `dims`. `operands` are evaluated by
  // the emitter (fusion members inline). Writes `outs` (kept-dims shape) or,
  // when `splits` > 1, partial results laid out [split][kept].
  // Several reductions over the same index space (same input shape and dimensions) can share one kernel:
  // each part keeps its own accumulators, initial values and combiner; inputs common to the parts are read once.
  struct ReducePart {
    std::vector<Value*> operands;      // values reduced
    std::vector<Value*> inits;
    Block* body = nullptr;
    std::vector<DT> dts;
  };
  struct ReduceGen {
    std::vector<ReducePart> parts;
    std::vector<int64_t> in_shape, dims;
  };

  // `epilogue`: pointwise groups over the kept index space that are evaluated by the thread holding the final
  // value of each output (second pass of a split reduction only); `bound_results` are the reduce results their
  // expressions refer to, in accumulator order.
  static bool use_col4(int64_t Nk) { return Nk % 4 == 0 && Nk >= 64 && !getenv("B200_NO_COL4"); }

  Launch gen_reduce_kernel(const ReduceGen& rg, std::function<bool(Op*)> internal, int splits, bool col,
                           std::vector<Value*> outs, const std::vector<Group*>* epilogue = nullptr,
                           const std::vector<Value*>* bound_results = nullptr, BlockState* est = nullptr) {
    size_t n = 0;
    std::vector<DT> dts;
    std::vector<Value*> all_inits;
    for (auto& part : rg.parts) {
      n += part.operands.size();
      dts.insert(dts.end(), part.dts.begin(), part.dts.end());
      all_inits.insert(all_inits.end(), part.inits.begin(), part.inits.end());
    }
    std::vector<int64_t> kept_dims, kept_shape, red_shape;
    for (size_t d = 0; d < rg.in_shape.size(); d++) {
      if (std::find(rg.dims.begin(), rg.dims.end(), (int64_t)d) == rg.dims.end()) {
        kept_dims.push_back(d);
        kept_shape.push_back(rg.in_shape[d]);
      } else red_shape.push_back(rg.in_shape[d]);
    }
    int64_t Nk = 1, Nr = 1;
    for (auto s : kept_shape) Nk *= s;
    for (auto s : red_shape) Nr *= s;
    Emitter em;
    em.is_internal = internal;
    em.round_small_floats = true;
    int64_t total = Nk * std::max<int64_t>(Nr, 1);
    em.idx_t = total >= (1LL << 31) - 65536 ? "i64" : "int";
    em.indent_ = 6;
    // contexts
    Ctx kc;
    kc.shape = kept_shape;
    kc.lin = "o";
    Ctx rc;
    rc.shape = red_shape;
    rc.lin = "r";
    std::ostringstream pre;       // code before the loop (kept index decomposition, init loads)
    Emitter pe;
    pe.is_internal = [](Op*) { return false; };
    pe.idx_t = em.idx_t;
    pe.name_prefix = "k";
    pe.indent_ = 4;
    pe.ensure_idx(kc);
    // the emitter for the loop body needs the kept index names; reduced ones are computed inside
    em.ensure_idx(rc);
    Ctx oc;
    oc.shape = rg.in_shape;
    oc.idx.resize(rg.in_shape.size());
    {
      size_t ki = 0, ri = 0;
      for (size_t d = 0; d < rg.in_shape.size(); d++) {
        if (std::find(rg.dims.begin(), rg.dims.end(), (int64_t)d) == rg.dims.end()) oc.idx[d] = kc.idx[ki++];
        else oc.idx[d] = rc.idx[ri++];
      }
    }
    std::vector<std::string> vals;
    for (auto& part : rg.parts)
      for (auto* v : part.operands) vals.push_back(em.emit(v, oc));
    // combine(acc, val), part by part
    em.round_small_floats = false;
    {
      size_t base = 0;
      for (auto& part : rg.parts) {
        const size_t np = part.operands.size();
        std::vector<std::string> args;
        for (size_t k = 0; k < np; k++) args.push_back("acc" + std::to_string(base + k));
        for (size_t k = 0; k < np; k++) args.push_back(vals[base + k]);
        auto comb = em.emit_scalar_region(part.body, args);
        for (size_t k = 0; k < np; k++) em.line("acc" + std::to_string(base + k) + " = " + comb[k] + ";");
        base += np;
      }
    }
    // a second emitter instance renders combine(acc, other) for the cross-thread tree
    auto tree_combine = [&](Emitter& te, const std::string& other_prefix) {
      te.round_small_floats = false;
      size_t base = 0;
      for (auto& part : rg.parts) {
        const size_t np = part.operands.size();
        std::vector<std::string> a2;
        for (size_t k = 0; k < np; k++) a2.push_back("acc" + std::to_string(base + k));
        for (size_t k = 0; k < np; k++) a2.push_back(other_prefix + std::to_string(base + k));
        auto c2 = te.emit_scalar_region(part.body, a2);
        for (size_t k = 0; k < np; k++) te.line("acc" + std::to_string(base + k) + " = " + c2[k] + ";");
        base += np;
      }
    };
    // kernel parameters: outputs, then loop inputs, then init values
    std::vector<Value*> ins = em.inputs;
    std::vector<std::string> init_names;
    for (size_t k = 0; k < n; k++) {
      Value* iv = all_inits[k];
      Op* d = iv->def;
      if (d && d->short_name() == "constant") {
        DenseValue dv = attr_dense(d->attr("value"));
        init_names.push_back(literal(dv.type.dt, dv.data.data()));
      } else {
        size_t pos = std::find(ins.begin(), ins.end(), iv) - ins.begin();
        if (pos == ins.size()) ins.push_back(iv);
        std::string e = "in" + std::to_string(pos) + "[0]";
        if (iv->type.dt == DT::BF16) e = "bf16_to_f(" + e + ")";
        else if (iv->type.dt == DT::F16) e = "f16_to_f(" + e + ")";
        else if (iv->type.dt == DT::PRED) e = "(" + e + " != 0)";
        init_names.push_back(e);
      }
    }
    // epilogue code (before the signature is printed: it adds outputs and inputs)
    std::string epi;
    if (epilogue && !epilogue->empty()) {
      Emitter ee;
      ee.idx_t = em.idx_t;
      ee.name_prefix = "e";
      ee.indent_ = 4;
      ee.seed_inputs(ins);
      for (size_t k = 0; k < bound_results->size(); k++) ee.bound[(*bound_results)[k]] = "acc" + std::to_string(k);
      ee.is_internal = [&](Op* o) {
        for (Group* eg : *epilogue) if (eg->members.count(o)) return true;
        return is_dup(o) && !est->dup_materialize.count(o) && !slot_of.count(o->results[0]);
      };
      Ctx ec;
      ec.shape = kept_shape;
      ec.lin = "o";
      ee.ensure_idx(ec);
      std::vector<std::pair<Value*, std::string>> stores;
      for (Group* eg : *epilogue)
        for (Op* r : eg->roots) stores.push_back({r->results[0], ee.emit(r->results[0], ec)});
      for (auto& st2 : stores) {
        ee.line("out" + std::to_string(outs.size()) + "[o] = " + store_expr(st2.first->type.dt, st2.second) + ";");
        outs.push_back(st2.first);
      }
      epi = ee.str();
      ins = ee.inputs;
    }
    std::ostringstream src;
    const char* it = em.idx_t.c_str();
    Launch L;
    L.outs = outs;
    L.ins = ins;
    const bool col4 = col && use_col4(Nk);
    if (col4) {
      // Column strategy with four consecutive kept indices per thread: four times the bytes in flight per thread
      // and, for inputs read at their own position, neighbouring loads the compiler can merge into 16-byte ones
      // (every slot and buffer starts on a 256-byte boundary). The per-index code is the scalar one, instantiated
      // four times with the accumulators indexed by q.
      const int TX = (int)std::min<int64_t>(32, Nk / 4), TY = 256 / TX;
      const int unroll_r = 2;      // measured on the ResNet18 step: 1 -> 5.20 ms, 2 -> 5.15, 4 -> 5.18 (scalar form 5.21)
      auto per_q = [](std::string text) {
        return std::regex_replace(text, std::regex("\\bacc(\\d+)\\b"), "acc$1[q]");
      };
      src << "extern \"C\" __global__ void __launch_bounds__(256) @NAME@(" << signature(outs, ins) << ") {\n";
      for (size_t k = 0; k < ins.size(); k++)
        if (dt_size(ins[k]->type.dt) == 4 && ins[k]->type.numel() % 4 == 0)
          src << "  in" << k << " = (const " << s_type(ins[k]->type.dt) << "*)__builtin_assume_aligned(in" << k << ", 16);\n";
      for (size_t k = 0; k < n; k++)
        src << "  __shared__ " << c_type(dts[k]) << " sm" << k << "[" << TY << "][" << TX * 4 + 4 << "];\n";
      src << "  const " << it << " o4 = ((" << it << ")blockIdx.x * " << TX << " + threadIdx.x) * 4;\n";
      src << "  const bool live = o4 < (" << it << ")" << Nk << "LL;\n";
      for (size_t k = 0; k < n; k++)
        src << "  " << c_type(dts[k]) << " acc" << k << "[4] = {" << init_names[k] << ", " << init_names[k] << ", "
            << init_names[k] << ", " << init_names[k] << "};\n";
      src << "  if (live) {\n";
      src << "    #pragma unroll " << unroll_r << "\n";
      src << "    for (" << it << " r = (" << it << ")blockIdx.y * " << TY << " + threadIdx.y; r < (" << it << ")" << Nr
          << "LL; r += " << TY << " * (" << it << ")gridDim.y) {\n";
      src << "      #pragma unroll\n      for (int q = 0; q < 4; ++q) {\n        const " << it << " o = o4 + q;\n";
      src << pe.str() << per_q(em.str());
      src << "      }\n    }\n  }\n";
      src << "  #pragma unroll\n  for (int q = 0; q < 4; ++q) {\n";
      for (size_t k = 0; k < n; k++) src << "    sm" << k << "[threadIdx.y][threadIdx.x * 4 + q] = acc" << k << "[q];\n";
      src << "  }\n  __syncthreads();\n";
      src << "  if (threadIdx.y == 0 && live) {\n";
      src << "    #pragma unroll\n    for (int q = 0; q < 4; ++q) {\n      const " << it << " o = o4 + q;\n";
      src << "      for (int y = 1; y < " << TY << "; ++y) {\n";
      for (size_t k = 0; k < n; k++)
        src << "        const " << c_type(dts[k]) << " oth" << k << " = sm" << k << "[y][threadIdx.x * 4 + q];\n";
      {
        Emitter te;
        te.idx_t = em.idx_t;
        te.name_prefix = "t";
        te.indent_ = 8;
        tree_combine(te, "oth");
        src << per_q(te.str());
      }
      src << "      }\n";
      for (size_t k = 0; k < n; k++)
        src << "      out" << k << "[(" << it << ")blockIdx.y * " << Nk << " + o] = "
            << store_expr(outs[k]->type.dt, "acc" + std::to_string(k) + "[q]") << ";\n";
      src << per_q(epi);
      src << "    }\n  }\n}\n";
      L.grid[0] = (unsigned)((Nk + TX * 4 - 1) / (TX * 4)); L.grid[1] = (unsigned)splits; L.grid[2] = 1;
      L.block[0] = TX; L.block[1] = TY; L.block[2] = 1;
    } else if (col) {
      // threads along the kept index (coalesced), rows of the reduced range over threadIdx.y and blockIdx.y
      const int TX = 32, TY = 8;
      src << "extern \"C\" __global__ void __launch_bounds__(" << TX * TY << ") @NAME@(" << signature(outs, ins) << ") {\n";
      for (size_t k = 0; k < n; k++)
        src << "  __shared__ " << c_type(dts[k]) << " sm" << k << "[" << TY << "][" << TX + 1 << "];\n";
      src << "  const " << it << " o = (" << it << ")blockIdx.x * " << TX << " + threadIdx.x;\n";
      src << "  const bool live = o < (" << it << ")" << Nk << "LL;\n";
      for (size_t k = 0; k < n; k++) src << "  " << c_type(dts[k]) << " acc" << k << " = " << init_names[k] << ";\n";
      src << "  if (live) {\n" << pe.str();
      src << "    #pragma unroll 4\n";      // independent loads of several rows in flight per thread
      src << "    for (" << it << " r = (" << it << ")blockIdx.y * " << TY << " + threadIdx.y; r < (" << it << ")" << Nr
          << "LL; r += " << TY << " * (" << it << ")gridDim.y) {\n";
      src << em.str();
      src << "    }\n  }\n";
      for (size_t k = 0; k < n; k++) src << "  sm" << k << "[threadIdx.y][threadIdx.x] = acc" << k << ";\n";
      src << "  __syncthreads();\n";
      src << "  if (threadIdx.y == 0 && live) {\n";
      src << "    for (int y = 1; y < " << TY << "; ++y) {\n";
      for (size_t k = 0; k < n; k++)
        src << "      const " << c_type(dts[k]) << " oth" << k << " = sm" << k << "[y][threadIdx.x];\n";
      Emitter te;
      te.idx_t = em.idx_t;
      te.name_prefix = "t";
      te.indent_ = 6;
      tree_combine(te, "oth");
      src << te.str();
      src << "    }\n";
      for (size_t k = 0; k < n; k++)
        src << "    out" << k << "[(" << it << ")blockIdx.y * " << Nk << " + o] = "
            << store_expr(outs[k]->type.dt, "acc" + std::to_string(k)) << ";\n";
      src << epi;
      src << "  }\n}\n";
      L.grid[0] = (unsigned)((Nk + TX - 1) / TX); L.grid[1] = (unsigned)splits; L.grid[2] = 1;
      L.block[0] = TX; L.block[1] = TY; L.block[2] = 1;
    } else {
      // T threads cooperate on one output; the reduced range is contiguous-ish along threads
      // a block per output from 128 reduced elements on: second passes over a few hundred partial rows are latency-
      // bound, and 256 threads fetch them in one or two rounds of loads where a warp would need ten to twenty
      int T = Nr >= 128 ? 256 : 32;
      int per_block = 256 / T;
      src << "extern \"C\" __global__ void __launch_bounds__(256) @NAME@(" << signature(outs, ins) << ") {\n";
      if (T == 256)
        for (size_t k = 0; k < n; k++) src << "  __shared__ " << c_type(dts[k]) << " sm" << k << "[8];\n";
      src << "  const " << it << " o = (" << it << ")blockIdx.x * " << per_block << " + threadIdx.x / " << T << ";\n";
      src << "  const int lane = threadIdx.x % " << T << ";\n";
      src << "  const bool live = o < (" << it << ")" << Nk << "LL;\n";
      for (size_t k = 0; k < n; k++) src << "  " << c_type(dts[k]) << " acc" << k << " = " << init_names[k] << ";\n";
      src << "  if (live) {\n" << pe.str();
      src << "    #pragma unroll 4\n";
      src << "    for (" << it << " r = (" << it << ")blockIdx.y * " << T << " + lane; r < (" << it << ")" << Nr
          << "LL; r += " << T << " * (" << it << ")gridDim.y) {\n";
      src << em.str();
      src << "    }\n  }\n";
      src << "  #pragma unroll\n  for (int m = 16; m >= 1; m >>= 1) {\n";
      for (size_t k = 0; k < n; k++)
        src << "    const " << c_type(dts[k]) << " oth" << k << " = shfl_xor(acc" << k << ", m);\n";
      {
        Emitter te;
        te.idx_t = em.idx_t;
        te.name_prefix = "t";
        te.indent_ = 4;
        tree_combine(te, "oth");
        src << te.str();
      }
      src << "  }\n";
      if (T == 256) {
        src << "  const int warp = threadIdx.x / 32;\n";
        src << "  if ((threadIdx.x & 31) == 0) {";
        for (size_t k = 0; k < n; k++) src << " sm" << k << "[warp] = acc" << k << ";";
        src << " }\n  __syncthreads();\n";
        src << "  if (threadIdx.x == 0) {\n    for (int w = 1; w < 8; ++w) {\n";
        for (size_t k = 0; k < n; k++)
          src << "      const " << c_type(dts[k]) << " oth" << k << " = sm" << k << "[w];\n";
        Emitter te;
        te.idx_t = em.idx_t;
        te.name_prefix = "u";
        te.indent_ = 6;
        tree_combine(te, "oth");
        src << te.str();
        src << "    }\n  }\n";
      }
      src << "  if (lane == 0 && live) {\n";
      for (size_t k = 0; k < n; k++)
        src << "    out" << k << "[(" << it << ")blockIdx.y * " << Nk << " + o] = "
            << store_expr(outs[k]->type.dt, "acc" + std::to_string(k)) << ";\n";
      src << epi;
      src << "  }\n}\n";
      L.grid[0] = (unsigned)((Nk + per_block - 1) / per_block); L.grid[1] = (unsigned)splits; L.grid[2] = 1;
      L.block[0] = 256; L.block[1] = L.block[2] = 1;
    }
    L.kernel = add_kernel(src.str(), "reduce");
    return L;
  }

  // ---- implicit GEMM lowering ----------------------------------------------------
  struct RowEnt { long long off; int h0, w0; };
  struct ColEnt { long long off; int dh, dw; };

  static std::vector<int64_t> strides_of(const std::vector<int64_t>& dims) {
    std::vector<int64_t> s(dims.size());
    int64_t st = 1;
    for (int d = (int)dims.size() - 1; d >= 0; d--) { s[d] = st; st *= dims[d]; }
    return s;
  }

  // Split the contraction over blockIdx.z when the output has too few tiles to fill the GPU. A small cost model
  // (measured on the ResNet layer shapes: about 0.6 us per 128 x 64 x 32 k-tile, 0.9 us per 128 x 128 x 32 one,
  // 6 us of fixed cost per wave of CTAs, partial sums written and re-read at about 3 TB/s) picks the split
  // that minimises waves * time per CTA + reduction time.
  void choose_split_k(IGemmParams& p) {
    const int bn = p.N >= 128 ? 128 : 64;
    const long long tiles = (long long)((p.M + 127) / 128) * ((p.N + bn - 1) / bn) * p.groups;
    const long long ktiles = (p.K + 31) / 32;
    // the scalar-gather kernel (operands without 16-byte structure) spends about 10 us per k-tile and runs two
    // CTAs per SM; the row-gather kernels one CTA per SM
    // 64-wide row-gather tiles run as two half-size CTAs per SM (about 1 us per k-tile each, two at a time)
    const bool half = p.vec && p.seg && bn == 64;
    const double tile_us = !p.vec ? 10.0 : (bn == 128 ? 0.9 : (half ? 1.0 : 0.6));
    const long long per_wave = (!p.vec || half) ? 296 : 148;
    int best = 1;
    double best_cost = 1e30;
    // a split keeps at least 8 k-tiles, except when the output has so few tiles that even then most of the GPU
    // would idle (the small products of a recurrent cell): those go down to 2 k-tiles per CTA
    const long long min_kt = tiles * 8 <= per_wave ? 2 : 8;
    const int max_split = (int)std::min<long long>(592, std::max<long long>(1, ktiles / min_kt));
    for (int split = 1; split <= max_split; split++) {
      const long long waves = (tiles * split + per_wave - 1) / per_wave;
      const long long kt = (ktiles + split - 1) / split;
      double cost = (double)waves * ((double)kt * tile_us + 6.0);
      if (split > 1) cost += 3.0 + 2.0 * split * (double)p.M * p.N * p.groups * 4.0 / 3e6;
      if (cost < best_cost * 0.97) { best_cost = cost; best = split; }
    }
    p.split_k = best;
  }

  Step lower_conv(Op* op, BlockState& st) {
    Value *lhs = op->operands[0], *rhs = op->operands[1], *out = op->results[0];
    if (lhs->type.dt != DT::F32 || rhs->type.dt != DT::F32 || out->type.dt != DT::F32)
      throw CompileError("stablehlo.convolution: only f32 operands are supported so far, got " + lhs->type.str());
    std::string dn = op->attr("dimension_numbers");
    // '#stablehlo.conv<[b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f]>' (also accepts the 'raw' keyword-less form)
    auto parse_spec = [&](const std::string& s) {
      std::vector<std::string> toks;
      std::string cur;
      for (char c : s) {
        if (c == ',' ) { toks.push_back(cur); cur.clear(); }
        else if (!isspace((unsigned char)c)) cur += c;
      }
      if (!cur.empty()) toks.push_back(cur);
      return toks;
    };
    size_t a0 = dn.find('['), a1 = dn.find(']', a0);
    size_t b0 = dn.find('[', a1), b1 = dn.find(']', b0);
    size_t c0 = dn.find('[', b1), c1 = dn.find(']', c0);
    if (a0 == std::string::npos || c1 == std::string::npos) throw CompileError("convolution: cannot read dimension_numbers");
    auto ls = parse_spec(dn.substr(a0 + 1, a1 - a0 - 1));
    auto rs = parse_spec(dn.substr(b0 + 1, b1 - b0 - 1));
    auto os = parse_spec(dn.substr(c0 + 1, c1 - c0 - 1));
    if (ls.size() != 4 && ls.size() != 3) throw CompileError("convolution: only 1 or 2 spatial dimensions are supported");
    const bool one_d = ls.size() == 3;
    auto pos = [&](const std::vector<std::string>& spec, const std::string& c) -> int {
      for (size_t k = 0; k < spec.size(); k++)
        if (spec[k] == c) return (int)k;
      throw CompileError("convolution: dimension_numbers lacks '" + c + "'");
    };
    auto get2 = [&](const char* name, int64_t dflt) {
      std::vector<int64_t> v = op->has(name) ? attr_i64s(op->attr(name)) : std::vector<int64_t>{};
      if (v.empty()) v = {dflt, dflt};
      if (v.size() == 1) v.push_back(dflt);
      return v;
    };
    auto stride = get2("window_strides", 1), ldil = get2("lhs_dilation", 1), rdil = get2("rhs_dilation", 1);
    std::vector<int64_t> pad = {0, 0, 0, 0};
    if (op->has("padding")) pad = attr_i64s(op->attr("padding"));
    while (pad.size() < 4) pad.push_back(0);
    if (op->has("window_reversal")) {
      std::string wr = op->attr("window_reversal");
      if (wr.find("true") != std::string::npos) throw CompileError("convolution: window_reversal is not supported");
    }
    int64_t G = op->has("feature_group_count") ? attr_int(op->attr("feature_group_count")) : 1;
    int64_t BG = op->has("batch_group_count") ? attr_int(op->attr("batch_group_count")) : 1;
    if (BG > 1 && G > 1) throw CompileError("convolution: feature_group_count and batch_group_count cannot both exceed 1");
    auto sl = strides_of(lhs->type.dims), sr = strides_of(rhs->type.dims), so = strides_of(out->type.dims);
    int lb = pos(ls, "b"), lf = pos(ls, "f"), l0 = pos(ls, "0"), l1 = one_d ? -1 : pos(ls, "1");
    int ro = pos(rs, "o"), ri = pos(rs, "i"), r0 = pos(rs, "0"), r1 = one_d ? -1 : pos(rs, "1");
    int ob = pos(os, "b"), of = pos(os, "f"), o0 = pos(os, "0"), o1 = one_d ? -1 : pos(os, "1");
    auto dim_or1 = [](const TensorType& t, int d) -> int64_t { return d < 0 ? 1 : t.dims[d]; };
    auto str_or0 = [](const std::vector<int64_t>& s, int d) -> int64_t { return d < 0 ? 0 : s[d]; };
    int64_t Nb = lhs->type.dims[lb] / BG, Cin = lhs->type.dims[lf], H = lhs->type.dims[l0], W = dim_or1(lhs->type, l1);
    int64_t KH = rhs->type.dims[r0], KW = dim_or1(rhs->type, r1), Cg = rhs->type.dims[ri], O = rhs->type.dims[ro];
    int64_t OH = out->type.dims[o0], OW = dim_or1(out->type, o1);
    const int64_t groups = std::max(G, BG);
    if (Cin != Cg * G || O % groups) throw CompileError("convolution: inconsistent feature groups");
    int64_t Og = O / groups;
    const int64_t sl1 = str_or0(sl, l1), sr1 = str_or0(sr, r1), so1 = str_or0(so, o1);
    IGemmParams p;
    p.M = (int)(Nb * OH * OW);
    p.N = (int)Og;
    p.K = (int)(KH * KW * Cg);
    p.groups = (int)groups;
    p.Hd = (int)(H == 0 ? 0 : (H - 1) * ldil[0] + 1);
    p.Wd = (int)(W == 0 ? 0 : (W - 1) * ldil[1] + 1);
    p.ldh = (int)ldil[0];
    p.ldw = (int)ldil[1];
    p.a_sh = sl[l0];
    p.a_sw = sl1;
    p.needs_mask = 1;
    bool batch_fastest = sl[lb] == 1 && sl[lf] != 1;
    std::vector<RowEnt> arow(p.M);
    std::vector<long long> crow(p.M);
    for (int64_t m = 0; m < p.M; m++) {
      int64_t n, oh, ow;
      if (batch_fastest) { n = m % Nb; ow = (m / Nb) % OW; oh = m / (Nb * OW); }
      else { ow = m % OW; oh = (m / OW) % OH; n = m / (OW * OH); }
      arow[m] = {n * sl[lb], (int)(oh * stride[0] - pad[0]), (int)(ow * stride[1] - pad[2])};
      crow[m] = n * so[ob] + oh * so[o0] + ow * so1;
    }
    if (p.ldh > 1 || p.ldw > 1) {
      // Input dilation (the input gradient of a strided convolution): a window position only meets real input where
      // (h0 + dh) is a multiple of the dilation, so rows of one phase (h0 mod ldh, w0 mod ldw) share their live
      // window positions. Rows are visited phase by phase, which lets whole k-tiles be skipped per row tile
      // (make_igemm builds the list); the output addresses follow the rows, so the result is unchanged.
      auto phase = [&](const RowEnt& r) {
        const int ph = ((r.h0 % p.ldh) + p.ldh) % p.ldh, pw = ((r.w0 % p.ldw) + p.ldw) % p.ldw;
        return ph * p.ldw + pw;
      };
      std::vector<int64_t> order(p.M);
      for (int64_t m = 0; m < p.M; m++) order[m] = m;
      std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return phase(arow[a]) < phase(arow[b]); });
      std::vector<RowEnt> ar2(p.M);
      std::vector<long long> cr2(p.M);
      for (int64_t m = 0; m < p.M; m++) { ar2[m] = arow[order[m]]; cr2[m] = crow[order[m]]; }
      arow.swap(ar2);
      crow.swap(cr2);
    }
    std::vector<ColEnt> acol(p.K);
    std::vector<long long> bcol(p.K);
    bool rev0 = false, rev1 = false;              // kernel-spatial dimensions read back to front (folded stablehlo.reverse)
    if (op->has("b200.rhs_reversed"))
      for (auto d : attr_i64s(op->attr("b200.rhs_reversed"))) { rev0 = rev0 || d == r0; rev1 = rev1 || (!one_d && d == r1); }
    for (int64_t k = 0; k < p.K; k++) {
      int64_t c = k % Cg, kw = (k / Cg) % KW, kh = k / (Cg * KW);
      acol[k] = {c * sl[lf], (int)(kh * rdil[0]), (int)(kw * rdil[1])};
      bcol[k] = c * sr[ri] + (rev0 ? KH - 1 - kh : kh) * sr[r0] + (rev1 ? KW - 1 - kw : kw) * sr1;
    }
    std::vector<long long> bn(p.N), cn(p.N), ag(groups), bg(groups), cg(groups);
    for (int64_t n = 0; n < p.N; n++) { bn[n] = n * sr[ro]; cn[n] = n * so[of]; }
    for (int64_t g = 0; g < groups; g++) {
      // feature groups slice the input channels; batch groups slice the input batch (linalg.cc:339-362)
      ag[g] = BG > 1 ? g * Nb * sl[lb] : g * Cg * sl[lf];
      bg[g] = g * Og * sr[ro];
      cg[g] = g * Og * so[of];
    }
    p.a_contig = (sl[lf] == 1 && Cg > 1) ? 0 : (batch_fastest ? 1 : 0);
    p.b_contig = sr[ro] == 1 ? 0 : 1;
    // TMA feed of A: stride-1 two-dimensional convolution without input dilation over a dense NHWC input with a
    // multiple of 32 channels, output rows dividing the 128-row tile (make_igemm drops it again where the row gather
    // kernel with A in tensor memory is not the one that runs)
    if (!one_d && groups == 1 && stride[0] == 1 && stride[1] == 1 && p.ldh == 1 && p.ldw == 1 && !batch_fastest &&
        sl[lf] == 1 && sl1 == Cin && sl[l0] == W * Cin && sl[lb] == H * W * Cin && Cin % 32 == 0 && OW >= 1 && 128 % OW == 0 &&
        OW <= 256 && !getenv("B200_NO_TMA_A")) {
      const int64_t rows_per_tile = 128 / OW;                    // output rows in a tile
      const int64_t box_h = std::min<int64_t>(OH, rows_per_tile);
      const int64_t box_n = std::max<int64_t>(1, rows_per_tile / OH);
      const bool whole = OH % box_h == 0 && (box_n == 1 || OH * OW * box_n == 128) && (box_n == 1 || rows_per_tile % OH == 0);
      if (whole && box_h <= 256 && box_n <= 256 && H < (1 << 15) && W < (1 << 15)) {
        p.a_tma = 1;
        p.tma_c = (int)Cin; p.tma_w = (int)W; p.tma_h = (int)H; p.tma_n = (int)Nb;
        p.tma_ow = (int)OW; p.tma_oh = (int)OH; p.tma_box_h = (int)box_h; p.tma_box_n = (int)box_n;
        p.tma_kw = (int)KW; p.tma_pad_h = (int)pad[0]; p.tma_pad_w = (int)pad[2];
        p.tma_rdil_h = (int)rdil[0]; p.tma_rdil_w = (int)rdil[1];
      }
    }
    return make_igemm(op, p, lhs, rhs, out, arow, acol, bcol, bn, crow, cn, ag, bg, cg, st);
  }

  // dot_general on 16-bit operands: optional row repacks, then one GEMM16 step (args: A, B, C, [fp32 scratch],
  // [counters]; iparams: which of the two optional arguments are present).
  void lower_dot16(Op* op, const Dot16& d, Plan& plan, BlockState& st) {
    Value *lhs = op->operands[0], *rhs = op->operands[1], *out = op->results[0];
    auto operand = [&](Value* v, const Dot16::Repack& r) -> int {
      if (!r.needed) return slot_of.at(v);
      auto key = std::make_tuple(st.block, v, r.dst_ld);
      auto it = repacked.find(key);
      if (it != repacked.end()) return it->second;
      TensorType t;
      t.dt = v->type.dt;
      t.dims = {(int64_t)r.rows, (int64_t)r.dst_ld};
      const int tmp = new_slot(Slot::TEMP, t, st.arena);
      Step c;
      c.kind = Step::REPACK16;
      c.label = "row repack for " + op->name;
      c.args = {tmp, slot_of.at(v)};
      c.iparams = {r.rows, r.cols, r.dst_ld, r.src_ld};
      plan.steps.push_back(std::move(c));
      repacked[key] = tmp;
      return tmp;
    };
    Step s;
    s.kind = Step::GEMM16;
    s.label = op->name;
    s.g16 = d.g;
    // B may be read ahead of the wait for the kernel in front when that kernel cannot be its writer: B is a program
    // input, or it was made in front of the loop whose body this is and a kernel of the body already precedes this one
    {
      bool is_static = false;
      if (!d.rb.needed) {
        if (!rhs->def) is_static = rhs->owner && rhs->owner->parent_op == nullptr;
        else if (rhs->def->parent != st.block) {
          for (auto& prev : plan.steps)
            if (prev.kind == Step::KERNEL || prev.kind == Step::GEMM16 || prev.kind == Step::IGEMM) { is_static = true; break; }
        }
      }
      s.g16.b_static = is_static ? 1 : 0;
    }
    const int a = operand(lhs, d.ra), b = operand(rhs, d.rb);
    s.args = {a, b, slot_of.at(out)};
    s.iparams = {0, 0};
    if (d.g.scratch_floats > 0) {
      TensorType t;
      t.dt = DT::F32;
      t.dims = {(int64_t)d.g.scratch_floats};
      s.args.push_back(new_slot(Slot::TEMP, t, st.arena));
      s.iparams[0] = 1;
    }
    if (d.g.counters > 0) {
      std::vector<int> zeros((size_t)d.g.counters, 0);
      s.args.push_back(table_slot(zeros.data(), zeros.size() * sizeof(int)));
      s.iparams[1] = 1;
    }
    plan.steps.push_back(std::move(s));
  }
  std::map<std::tuple<Block*, Value*, long long>, int> repacked;   // padded copies of operands, per block

  Step lower_dot(Op* op, BlockState& st) {
    Value *lhs = op->operands[0], *rhs = op->operands[1], *out = op->results[0];
    if (lhs->type.dt != DT::F32 || rhs->type.dt != DT::F32 || out->type.dt != DT::F32)
      throw CompileError("stablehlo.dot_general: only f32 operands are supported so far, got " + lhs->type.str());
    auto f = attr_struct(op->attr("dot_dimension_numbers"));
    auto lbd = f["lhs_batching_dimensions"], rbd = f["rhs_batching_dimensions"];
    auto lcd = f["lhs_contracting_dimensions"], rcd = f["rhs_contracting_dimensions"];
    auto in = [](const std::vector<int64_t>& v, int64_t x) { return std::find(v.begin(), v.end(), x) != v.end(); };
    std::vector<int64_t> lfree, rfree;
    for (int d = 0; d < lhs->type.rank(); d++) if (!in(lbd, d) && !in(lcd, d)) lfree.push_back(d);
    for (int d = 0; d < rhs->type.rank(); d++) if (!in(rbd, d) && !in(rcd, d)) rfree.push_back(d);
    auto sl = strides_of(lhs->type.dims), sr = strides_of(rhs->type.dims);
    auto extent = [](const std::vector<int64_t>& dims, const std::vector<int64_t>& which) {
      int64_t n = 1;
      for (auto d : which) n *= dims[d];
      return n;
    };
    int64_t G = extent(lhs->type.dims, lbd), M = extent(lhs->type.dims, lfree), K = extent(lhs->type.dims, lcd),
            N = extent(rhs->type.dims, rfree);
    // offset of the multi-index (row-major over `which`) in a tensor with strides s
    auto offsets = [](const std::vector<int64_t>& dims, const std::vector<int64_t>& s, const std::vector<int64_t>& which,
                      int64_t count) {
      std::vector<long long> out(count);
      for (int64_t i = 0; i < count; i++) {
        int64_t rem = i;
        long long off = 0;
        for (int q = (int)which.size() - 1; q >= 0; q--) {
          int64_t dsz = dims[which[q]];
          off += (rem % dsz) * s[which[q]];
          rem /= dsz;
        }
        out[i] = off;
      }
      return out;
    };
    IGemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K; p.groups = (int)G;
    p.needs_mask = 0;
    auto am = offsets(lhs->type.dims, sl, lfree, M), ak = offsets(lhs->type.dims, sl, lcd, K);
    auto bk = offsets(rhs->type.dims, sr, rcd, K), bn = offsets(rhs->type.dims, sr, rfree, N);
    auto ag = offsets(lhs->type.dims, sl, lbd, G), bg = offsets(rhs->type.dims, sr, rbd, G);
    std::vector<RowEnt> arow(M);
    std::vector<ColEnt> acol(K);
    std::vector<long long> crow(M), cn(N), cg(G);
    for (int64_t m = 0; m < M; m++) { arow[m] = {am[m], 0, 0}; crow[m] = m * N; }
    for (int64_t k = 0; k < K; k++) acol[k] = {ak[k], 0, 0};
    for (int64_t n = 0; n < N; n++) cn[n] = n;
    for (int64_t g = 0; g < G; g++) cg[g] = g * M * N;
    p.a_contig = (K > 1 && ak[1] == 1) ? 0 : ((M > 1 && am[1] == 1) ? 1 : 0);
    p.b_contig = (N > 1 && bn[1] == 1) ? 0 : 1;
    return make_igemm(op, p, lhs, rhs, out, arow, acol, bk, bn, crow, cn, ag, bg, cg, st);
  }

  Step make_igemm(Op* op, IGemmParams p, Value* lhs, Value* rhs, Value* out, const std::vector<RowEnt>& arow,
                  const std::vector<ColEnt>& acol, const std::vector<long long>& bcol, const std::vector<long long>& bn,
                  const std::vector<long long>& crow, const std::vector<long long>& cn, const std::vector<long long>& ag,
                  const std::vector<long long>& bg, const std::vector<long long>& cg, BlockState& st) {
    // Can the operands be gathered 16 bytes at a time? A chunk is four consecutive contraction indices of one
    // row (K-major storage) or four consecutive rows at one contraction index (MN-major storage); it must be
    // four consecutive, 16-byte aligned floats that share one convolution-window position.
    auto a_kmajor_ok = [&]() {
      if (p.K % 4) return false;
      for (int k = 0; k < p.K; k += 4) {
        if (acol[k].off % 4) return false;
        for (int i = 1; i < 4; i++)
          if (acol[k + i].off != acol[k].off + i || acol[k + i].dh != acol[k].dh || acol[k + i].dw != acol[k].dw) return false;
      }
      for (auto& r : arow) if (r.off % 4) return false;
      return true;
    };
    auto a_mnmajor_ok = [&]() {
      if (p.M % 4) return false;
      for (int m = 0; m < p.M; m += 4) {
        if (arow[m].off % 4) return false;
        for (int i = 1; i < 4; i++)
          if (arow[m + i].off != arow[m].off + i || arow[m + i].h0 != arow[m].h0 || arow[m + i].w0 != arow[m].w0) return false;
      }
      for (auto& c : acol) if (c.off % 4) return false;
      return true;
    };
    auto b_kmajor_ok = [&]() {
      if (p.K % 4) return false;
      for (int k = 0; k < p.K; k += 4) {
        if (bcol[k] % 4) return false;
        for (int i = 1; i < 4; i++) if (bcol[k + i] != bcol[k] + i) return false;
      }
      for (auto v : bn) if (v % 4) return false;
      return true;
    };
    auto b_mnmajor_ok = [&]() {
      if (p.N % 4) return false;
      for (int n = 0; n < p.N; n += 4) {
        if (bn[n] % 4) return false;
        for (int i = 1; i < 4; i++) if (bn[n + i] != bn[n] + i) return false;
      }
      for (auto v : bcol) if (v % 4) return false;
      return true;
    };
    bool strides_ok = (!p.needs_mask || (p.a_sh % 4 == 0 && p.a_sw % 4 == 0));
    for (auto v : ag) strides_ok &= v % 4 == 0;
    for (auto v : bg) strides_ok &= v % 4 == 0;
    int a_major = -1, b_major = -1;        // 0: K-major, 1: MN-major
    if (strides_ok) {
      if (p.a_contig == 0 && a_kmajor_ok()) a_major = 0;
      else if (a_mnmajor_ok()) a_major = 1;
      else if (a_kmajor_ok()) a_major = 0;
      if (p.b_contig == 1 && b_kmajor_ok()) b_major = 0;
      else if (b_mnmajor_ok()) b_major = 1;
      else if (b_kmajor_ok()) b_major = 0;
    }
    const bool fits_int = lhs->type.numel() < (1LL << 31) && rhs->type.numel() < (1LL << 31);   // kernels use 32-bit offsets
    if (a_major >= 0 && b_major >= 0 && fits_int) {
      p.vec = 1;
      p.a_contig = a_major;
      p.b_contig = b_major == 0 ? 1 : 0;
      // Segment gather: every aligned run of 32 indices along an operand's contiguous dimension is 32 consecutive
      // floats at one window position, so a whole 128-byte tile row shares one address and one mask.
      auto a_run = [&](int i0) {
        for (int i = 1; i < 32; i++) {
          if (a_major == 0) { if (acol[i0 + i].off != acol[i0].off + i || acol[i0 + i].dh != acol[i0].dh || acol[i0 + i].dw != acol[i0].dw) return false; }
          else if (arow[i0 + i].off != arow[i0].off + i || arow[i0 + i].h0 != arow[i0].h0 || arow[i0 + i].w0 != arow[i0].w0) return false;
        }
        return true;
      };
      auto b_run = [&](int i0) {
        const auto& t = b_major == 0 ? bcol : bn;
        for (int i = 1; i < 32; i++) if (t[i0 + i] != t[i0] + i) return false;
        return true;
      };
      const int a_ext = a_major == 0 ? p.K : p.M, b_ext = b_major == 0 ? p.K : p.N;
      bool seg = p.K % 32 == 0 && a_ext % 32 == 0 && b_ext % 32 == 0;
      for (int i = 0; seg && i < a_ext; i += 32) seg = a_run(i);
      for (int i = 0; seg && i < b_ext; i += 32) seg = b_run(i);
      p.seg = seg ? 1 : 0;
    }
    p.c_vec = 1;
    for (size_t n = 1; n < cn.size(); n++) if (cn[n] != cn[0] + (long long)n) p.c_vec = 0;
    if (p.c_vec) {                                   // 2: every row of C also starts on a multiple of four floats
      bool al = !cn.empty() && cn[0] % 4 == 0;
      for (auto v : crow) al = al && v % 4 == 0;
      for (auto v : cg) al = al && v % 4 == 0;
      if (al) p.c_vec = 2;
    }
    if (!(p.seg && p.a_contig == 0)) p.a_tma = 0;
    choose_split_k(p);
    Step s;
    s.kind = Step::IGEMM;
    s.label = op->name;
    s.ig = p;
    auto tab = [&](const void* d, size_t n) { return table_slot(d, std::max<size_t>(n, 1)); };
    s.args = {slot_of.at(lhs), slot_of.at(rhs), slot_of.at(out),
              tab(arow.data(), arow.size() * sizeof(RowEnt)), tab(acol.data(), acol.size() * sizeof(ColEnt)),
              tab(bcol.data(), bcol.size() * 8), tab(bn.data(), bn.size() * 8), tab(crow.data(), crow.size() * 8),
              tab(cn.data(), cn.size() * 8), tab(ag.data(), ag.size() * 8), tab(bg.data(), bg.size() * 8),
              tab(cg.data(), cg.size() * 8)};
    if (p.split_k > 1) {
      TensorType t;
      t.dt = DT::F32;
      t.dims = {(int64_t)p.split_k, (int64_t)p.groups, (int64_t)p.M, (int64_t)p.N};
      s.args.push_back(new_slot(Slot::TEMP, t, st.arena));
    }
    if (p.seg && p.needs_mask && p.a_contig == 0 && p.split_k == 1 && p.groups == 1 && (p.ldh > 1 || p.ldw > 1)) {
      // per 128-row tile: the k-tiles in which at least one row meets real input (all 32 k of a tile share one
      // window position when the row gather applies)
      const int mtiles = (p.M + 127) / 128, ktiles = p.K / 32;
      std::vector<int> table((size_t)mtiles * (ktiles + 1), 0);
      long long kept = 0;
      for (int mt = 0; mt < mtiles; mt++) {
        int* row = &table[(size_t)mt * (ktiles + 1)];
        int cnt = 0;
        for (int kt = 0; kt < ktiles; kt++) {
          const ColEnt& c = acol[(size_t)kt * 32];
          bool live = false;
          for (int m = mt * 128; m < std::min(p.M, (mt + 1) * 128) && !live; m++) {
            const int ih = arow[m].h0 + c.dh, iw = arow[m].w0 + c.dw;
            live = ih >= 0 && iw >= 0 && ih < p.Hd && iw < p.Wd && ih % p.ldh == 0 && iw % p.ldw == 0;
          }
          if (live) row[1 + cnt++] = kt;
        }
        row[0] = cnt;
        kept += cnt;
      }
      if (kept < (long long)mtiles * ktiles) {
        s.ig.a_tma = 0;
        s.ig.kt_stride = ktiles;
        s.args.push_back(tab(table.data(), table.size() * sizeof(int)));
      }
    }
    return s;
  }

  // stablehlo.scatter in its general form (windows of any shape, point updates, batching dimensions;
  // src/pjrt_plugin/ops/gather_scatter.cc:296-699). A generated kernel turns every update element into the linear index of
  // the operand element it lands on (or a sentinel when its window does not fit, which drops the whole window), then
  // the pairs (destination, update element) are sorted by destination with the stable radix sort and every run is
  // applied in update order: deterministic like the row form.
  Step lower_scatter_general(Op* op, int kind, Plan& plan, BlockState& st) {
    Value *operand = op->operands[0], *indices = op->operands[1], *updates = op->operands[2], *out = op->results[0];
    auto f = attr_struct(op->attr("scatter_dimension_numbers"));
    const auto uwd = f["update_window_dims"], iwd = f["inserted_window_dims"], sdo = f["scatter_dims_to_operand_dims"];
    const auto ibd = f["input_batching_dims"], sbd = f["scatter_indices_batching_dims"];
    const int IR = indices->type.rank(), R = operand->type.rank(), UR = updates->type.rank();
    const int ivd = f.count("index_vector_dim") && !f["index_vector_dim"].empty() ? (int)f["index_vector_dim"][0] : IR;
    const int64_t U = updates->type.numel(), numel = operand->type.numel();
    if (U >= (1LL << 31) - 1024 || numel >= (1LL << 31) - 1) throw CompileError("stablehlo.scatter: more than 2^31 elements");
    auto has = [](const std::vector<int64_t>& v, int64_t x) { return std::find(v.begin(), v.end(), x) != v.end(); };
    std::vector<int> scatter_dims, window_dims, idx_batch_dims;
    for (int d = 0; d < UR; d++) if (!has(uwd, d)) scatter_dims.push_back(d);
    for (int d = 0; d < R; d++) if (!has(iwd, d) && !has(ibd, d)) window_dims.push_back(d);
    for (int d = 0; d < IR; d++) if (d != ivd) idx_batch_dims.push_back(d);
    if (window_dims.size() != uwd.size() || scatter_dims.size() != idx_batch_dims.size() || ibd.size() != sbd.size())
      throw CompileError("stablehlo.scatter: inconsistent scatter_dimension_numbers " + op->attr("scatter_dimension_numbers"));
    const int64_t ncomp = ivd < IR ? indices->type.dims[ivd] : 1;
    if ((int64_t)sdo.size() != ncomp) throw CompileError("stablehlo.scatter: scatter_dims_to_operand_dims does not match the index vector");
    TensorType t;
    t.dt = DT::I32;
    t.dims = {scatter_elems_scratch_ints(U)};
    const int scratch = new_slot(Slot::TEMP, t, st.arena);
    // ---- the key kernel
    Emitter em;
    em.is_internal = [](Op*) { return false; };
    em.idx_t = "int";
    em.indent_ = 2;
    Ctx root;
    root.shape = updates->type.dims;
    root.lin = "e";
    em.ensure_idx(root);
    auto uidx = [&](int d) { return root.idx[d]; };
    std::vector<int64_t> istr(IR, 1), ostr(R, 1);
    for (int d = IR - 2; d >= 0; d--) istr[d] = istr[d + 1] * indices->type.dims[d + 1];
    for (int d = R - 2; d >= 0; d--) ostr[d] = ostr[d + 1] * operand->type.dims[d + 1];
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(int* __restrict__ keys, const " << s_type(indices->type.dt)
        << "* __restrict__ idx) {\n";
    src << "  const int e = (int)blockIdx.x * " << kThreads << " + threadIdx.x;\n  if (e >= " << U << ") return;\n";
    src << em.str();
    // position of this update's index vector in the index tensor
    std::string ibase = "0LL";
    for (size_t k = 0; k < idx_batch_dims.size(); k++)
      ibase += " + (long long)" + uidx(scatter_dims[k]) + " * " + std::to_string(istr[idx_batch_dims[k]]) + "LL";
    src << "  const long long ib = " << ibase << ";\n";
    for (int d = 0; d < R; d++) src << "  long long f" << d << " = 0;\n";
    for (size_t k = 0; k < sdo.size(); k++)
      src << "  f" << sdo[k] << " = (long long)idx[ib + " << (ivd < IR ? (long long)k * istr[ivd] : 0LL) << "LL];\n";
    for (size_t q = 0; q < ibd.size(); q++) {
      const int pos = (int)(std::find(idx_batch_dims.begin(), idx_batch_dims.end(), (int)sbd[q]) - idx_batch_dims.begin());
      if (pos >= (int)scatter_dims.size()) throw CompileError("stablehlo.scatter: scatter_indices_batching_dims names the index vector dimension");
      src << "  f" << ibd[q] << " = (long long)" << uidx(scatter_dims[pos]) << ";\n";
    }
    src << "  bool ok = true;\n";
    for (int d = 0; d < R; d++) {
      int64_t wsize = 1;
      for (size_t k = 0; k < window_dims.size(); k++) if (window_dims[k] == d) wsize = updates->type.dims[uwd[k]];
      src << "  ok = ok && f" << d << " >= 0 && f" << d << " + " << wsize << " <= " << operand->type.dims[d] << ";\n";
    }
    for (size_t k = 0; k < window_dims.size(); k++) src << "  f" << window_dims[k] << " += (long long)" << uidx((int)uwd[k]) << ";\n";
    std::string dest = "0LL";
    for (int d = 0; d < R; d++) dest += " + f" + std::to_string(d) + " * " + std::to_string(ostr[d]) + "LL";
    src << "  keys[e] = ok ? (int)(" << dest << ") : " << numel << ";\n  keys[" << U << " + e] = e;\n}\n";
    Step ks;
    ks.kind = Step::KERNEL;
    ks.kernel = add_kernel(src.str(), "scatter_keys");
    ks.label = "scatter keys";
    ks.grid[0] = (unsigned)std::max<int64_t>(1, (U + kThreads - 1) / kThreads); ks.grid[1] = ks.grid[2] = 1;
    ks.block[0] = kThreads; ks.block[1] = ks.block[2] = 1;
    ks.args = {scratch, slot_of.at(indices)};
    ks.n_outs = 1;
    plan.steps.push_back(std::move(ks));
    Step s;
    s.kind = Step::SCATTER;
    s.label = op->name;
    s.dtype = operand->type.dt;
    s.bytes = operand->type.bytes();
    s.iparams = {numel, 1, U, 0, kind, 1};
    s.args = {slot_of.at(operand), slot_of.at(indices), slot_of.at(updates), slot_of.at(out), scratch};
    if (kind >= 0) return s;
    // The update computation as written (src/pjrt_plugin/ops/gather_scatter.cc:79-120 of the reference runs such a body
    // once over gathered values): the scatter step only sorts the pairs, then one thread per run of equal destinations
    // folds the run's updates into its element in update order through the compiled region.
    plan.steps.push_back(std::move(s));
    const int passes = (scatter_elems_launches(numel) - 1) / 3;
    const long long koff = (passes % 2) ? 2 * U : 0, ooff = (passes % 2) ? 3 * U : U;
    const char* ct = c_type(operand->type.dt);
    std::ostringstream as;
    as << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << s_type(operand->type.dt) << "* __restrict__ out0, const "
       << s_type(updates->type.dt) << "* __restrict__ in0, const int* __restrict__ scratch) {\n";
    as << "  const int* key = scratch + " << koff << "LL;\n  const int* order = scratch + " << ooff << "LL;\n";
    as << "  const int p = (int)blockIdx.x * " << kThreads << " + threadIdx.x;\n  if (p >= " << U << ") return;\n";
    as << "  const int dest = key[p];\n  if (dest >= " << numel << " || (p > 0 && key[p - 1] == dest)) return;\n";
    as << "  " << ct << " acc = " << load_expr(operand, "out0", "dest") << ";\n";
    as << "  for (int q = p; q < " << U << " && key[q] == dest; ++q) {\n";
    as << "    const " << ct << " upd = " << load_expr(updates, "in0", "order[q]") << ";\n";
    Emitter be;
    be.idx_t = "int";
    be.name_prefix = "b";
    be.indent_ = 4;
    be.round_small_floats = true;
    auto res = be.emit_scalar_region(op->regions[0].get(), {"acc", "upd"});
    if (res.size() != 1) throw CompileError("stablehlo.scatter: the update computation must return one value");
    as << be.str() << "    acc = " << res[0] << ";\n  }\n";
    as << "  out0[dest] = " << store_expr(operand->type.dt, "acc") << ";\n}\n";
    Step a;
    a.kind = Step::KERNEL;
    a.kernel = add_kernel(as.str(), "scatter_apply");
    a.label = "scatter apply";
    a.grid[0] = (unsigned)std::max<int64_t>(1, (U + kThreads - 1) / kThreads); a.grid[1] = a.grid[2] = 1;
    a.block[0] = kThreads; a.block[1] = a.block[2] = 1;
    a.args = {slot_of.at(out), slot_of.at(updates), scratch};
    a.n_outs = 1;
    return a;
  }

  // stablehlo.scatter in its row form (what jnp.take's gradient and x.at[idx].add(rows) lower to): the index
  // vector holds one coordinate along operand dimension 0 and every update is a whole row. Updates are applied
  // in update order per row with an fp32 accumulator, so the result is deterministic (src/pjrt_plugin/ops/gather_scatter.cc:296-699 handles the general form).
  Step lower_scatter(Op* op, Plan& plan, BlockState& st) {
    if (op->operands.size() != 3 || op->results.size() != 1)
      throw CompileError("stablehlo.scatter: only one operand / one update tensor is supported");
    Value *operand = op->operands[0], *indices = op->operands[1], *updates = op->operands[2], *out = op->results[0];
    auto f = attr_struct(op->attr("scatter_dimension_numbers"));
    const int ivd = f.count("index_vector_dim") && !f["index_vector_dim"].empty() ? (int)f["index_vector_dim"][0] : indices->type.rank() - 1;
    const auto uwd = f["update_window_dims"], iwd = f["inserted_window_dims"], sdo = f["scatter_dims_to_operand_dims"];
    const int R = operand->type.rank();
    bool ok = R >= 1 && iwd.size() == 1 && iwd[0] == 0 && sdo.size() == 1 && sdo[0] == 0 && f["input_batching_dims"].empty() &&
              ivd == indices->type.rank() - 1 && indices->type.dims.back() == 1 && (int)uwd.size() == R - 1;
    const int n_scatter = updates->type.rank() - (R - 1);
    for (int k = 0; ok && k < R - 1; k++)
      ok = uwd[k] == n_scatter + k && updates->type.dims[n_scatter + k] == operand->type.dims[k + 1];
    long long U = 1;
    for (int k = 0; ok && k < n_scatter; k++) {
      ok = k < indices->type.rank() - 1 && indices->type.dims[k] == updates->type.dims[k];
      U *= updates->type.dims[k];
    }
    Block* body = op->regions[0].get();
    int kind = -1;                                    // 0 assign, 1 add, 2 multiply, 3 minimum, 4 maximum
    if (body->ops.size() == 1 && body->ops[0]->operands.size() == 1 && body->ops[0]->operands[0] == body->args[1]) kind = 0;
    else if (body->ops.size() == 2) {
      const std::string sh = body->ops[0]->short_name();
      kind = sh == "add" ? 1 : sh == "multiply" ? 2 : sh == "minimum" ? 3 : sh == "maximum" ? 4 : -1;
    }
    DT dt = operand->type.dt;
    // any other update computation or element type: the general form with the computation compiled as it stands
    if (kind < 0 || !(dt == DT::F32 || dt == DT::BF16 || dt == DT::I32)) { kind = -1; ok = false; }
    if (updates->type.dt != dt || body->args.size() != 2) throw CompileError("stablehlo.scatter: malformed update computation");
    if (indices->type.dt != DT::I32 && indices->type.dt != DT::I64) throw CompileError("stablehlo.scatter: indices must be i32 or i64");
    ensure_slot(out, st);
    for (auto* o : op->operands)
      if (!slot_of.count(o)) throw CompileError("internal: operand of scatter has no storage");
    if (!ok) return lower_scatter_general(op, kind, plan, st);
    Step s;
    s.kind = Step::SCATTER;
    s.label = op->name;
    s.dtype = dt;
    s.bytes = operand->type.bytes();
    const long long rows = operand->type.dims[0];
    const long long row_elems = rows ? operand->type.numel() / rows : 0;
    s.iparams = {rows, row_elems, U, indices->type.dt == DT::I64 ? 8 : 4, kind};
    TensorType t;
    t.dt = DT::I32;
    t.dims = {scatter_rows_scratch_ints(rows, U)};
    s.args = {slot_of.at(operand), slot_of.at(indices), slot_of.at(updates), slot_of.at(out), new_slot(Slot::TEMP, t, st.arena)};
    return s;
  }

  // ---- block -> steps ----------------------------------------------------------------
  void ensure_slot(Value* v, BlockState& st) {
    if (slot_of.count(v)) return;
    if (v->type.dt == DT::TOKEN) {
      TensorType t;
      t.dt = DT::U8;
      slot_of[v] = new_slot(Slot::TEMP, t, st.arena);
      return;
    }
    slot_of[v] = new_slot(Slot::TEMP, v->type, st.arena);
  }

  void add_launch(Plan& plan, const Launch& L, const std::string& label, BlockState& st) {
    Step s;
    s.kind = Step::KERNEL;
    s.kernel = L.kernel;
    s.label = label;
    for (int k = 0; k < 3; k++) { s.grid[k] = L.grid[k]; s.block[k] = L.block[k]; }
    for (auto* o : L.outs) { ensure_slot(o, st); s.args.push_back(slot_of.at(o)); }
    s.n_outs = (int)L.outs.size();
    for (auto* i : L.ins) {
      if (!slot_of.count(i)) throw CompileError("internal: kernel input without storage: " + i->name + " (" + label + ")");
      s.args.push_back(slot_of.at(i));
    }
    plan.steps.push_back(std::move(s));
  }

  std::string group_label(Group* g) {
    std::map<std::string, int> cnt;
    for (auto* m : g->members) cnt[m->short_name()]++;
    std::string s = g->is_reduce ? "reduce_fusion{" : "fusion{";
    bool first = true;
    for (auto& kv : cnt) { s += (first ? "" : ",") + kv.first + (kv.second > 1 ? "x" + std::to_string(kv.second) : ""); first = false; }
    return s + "}";
  }


  // ---- row chains ------------------------------------------------------------------------
  // softmax, RMSNorm, LayerNorm and their gradients are chains of reductions over the trailing dimensions of one
  // tensor ("rows") and pointwise kernels over the same tensor that read the reductions' results through a broadcast
  // along the row (the reference matches these as named fusions: src/pjrt_plugin/passes/fuse_softmax.cc,
  // fuse_layer_norm.cc, fuse_rms_norm.cc). Such a chain becomes one kernel: a warp (rows under 128 elements) or a block
  // owns a row and runs the stages one after the other over it; a reduction's result stays in a register of every
  // thread, a pointwise value that only later stages read is recomputed instead of stored, and the row's operands come
  // from L1 / L2 after the first pass. Launches and round trips through memory drop by the length of the chain.
  struct RowChain {
    std::vector<Group*> stages;
    std::vector<int64_t> in_shape, kept_shape, red_shape;
    int64_t Nk = 1, Nr = 1;
  };

  bool row_form(Group* g, RowChain& rc) {
    if (!g->is_reduce || g->roots.empty()) return false;
    Op* r = g->roots[0];
    const auto& shape = r->operands[0]->type.dims;
    auto dims = attr_i64s(r->attr("dimensions"));
    std::sort(dims.begin(), dims.end());
    const int n = (int)shape.size(), nd = (int)dims.size();
    if (nd == 0 || nd > n) return false;
    for (int i = 0; i < nd; i++) if (dims[i] != n - nd + i) return false;      // a suffix of the dimensions
    rc.in_shape = shape;
    rc.kept_shape.assign(shape.begin(), shape.begin() + (n - nd));
    rc.red_shape.assign(shape.begin() + (n - nd), shape.end());
    rc.Nk = rc.Nr = 1;
    for (auto v : rc.kept_shape) rc.Nk *= v;
    for (auto v : rc.red_shape) rc.Nr *= v;
    if (rc.Nr < 32 || rc.Nr > 16384 || rc.Nk < 1 || rc.Nk * rc.Nr >= (1LL << 31)) return false;
    for (Op* root : g->roots) {
      if (root->operands[0]->type.dims != shape) return false;
      auto d2 = attr_i64s(root->attr("dimensions"));
      std::sort(d2.begin(), d2.end());
      if (d2 != dims) return false;
      const size_t np = root->operands.size() / 2;
      for (size_t k = np; k < root->operands.size(); k++) {
        Op* d = root->operands[k]->def;
        if (!(d && d->short_name() == "constant")) return false;
      }
    }
    return true;
  }

  // Can stage `g` run inside the chain? Every path from its outputs to a reduction result of the chain must keep the
  // row: elementwise operations at the full index, then one broadcast along the row from the kept shape.
  bool row_safe(Group* g, const RowChain& rc, const std::set<Op*>& members, const std::set<Value*>& reduced, BlockState& st) {
    enum { FULL, KEPT, OTHER };
    std::map<std::pair<Value*, int>, bool> memo;
    std::function<bool(Value*, int)> chk = [&](Value* v, int state) -> bool {
      if (reduced.count(v)) return state == KEPT || rc.Nk == 1;
      auto key = std::make_pair(v, state);
      auto it = memo.find(key);
      if (it != memo.end()) return it->second;
      memo[key] = true;
      Op* d = v->def;
      const bool internal = d && d->parent == st.block &&
                            (members.count(d) || (is_dup(d) && !st.dup_materialize.count(d) && !slot_of.count(v)));
      if (!internal) return true;                       // read from memory
      if (categorize(d) == Cat::REDUCE) return memo[key] = false;
      const std::string sh = d->short_name();
      bool ok = true;
      if (is_elementwise_op(sh)) {
        for (Value* o : d->operands) ok = ok && chk(o, o->type.dims == v->type.dims ? state : OTHER);
      } else if (sh == "broadcast_in_dim") {
        Value* o = d->operands[0];
        auto bd = attr_i64s(d->attr("broadcast_dimensions"));
        bool prefix = state == FULL && v->type.dims == rc.in_shape && o->type.dims == rc.kept_shape;
        for (size_t i = 0; i < bd.size() && prefix; i++) prefix = bd[i] == (int64_t)i;
        ok = chk(o, prefix ? KEPT : OTHER);
      } else {
        for (Value* o : d->operands) ok = ok && chk(o, OTHER);
      }
      return memo[key] = ok;
    };
    if (g->is_reduce) {
      for (Op* root : g->roots) {
        const size_t np = root->operands.size() / 2;
        for (size_t k = 0; k < np; k++) if (!chk(root->operands[k], FULL)) return false;
      }
      return true;
    }
    // a pointwise stage lives on the full index space or (the scalar arithmetic between a sum and its use) on the rows
    const bool kept = g->roots[0]->results[0]->type.dims != rc.in_shape;
    for (Op* root : g->roots) {
      if (root->results[0]->type.dims != (kept ? rc.kept_shape : rc.in_shape)) return false;
      if (!chk(root->results[0], kept ? KEPT : FULL)) return false;
    }
    return true;
  }

  // does `g` read (through its own members) a value of `produced`?
  bool reads_any(Group* g, const std::set<Value*>& produced, BlockState& st) {
    std::set<Value*> seen;
    std::function<bool(Value*)> walk = [&](Value* v) -> bool {
      if (produced.count(v)) return true;
      if (!seen.insert(v).second) return false;
      Op* d = v->def;
      if (!d || d->parent != st.block) return false;
      if (!(g->members.count(d) || (is_dup(d) && !st.dup_materialize.count(d) && !slot_of.count(v)))) return false;
      if (categorize(d) == Cat::REDUCE && !g->is_reduce) return false;
      for (Value* o : d->operands) if (walk(o)) return true;
      return false;
    };
    for (Op* m : g->members)
      for (Value* o : m->operands) if (walk(o)) return true;
    return false;
  }

  void emit_row_chain(const RowChain& rc, Plan& plan, BlockState& st) {
    const int64_t Nk = rc.Nk, Nr = rc.Nr;
    // rows of up to 1024 elements: a warp per row, eight rows per block (a block per row leaves most of its threads
    // without an element and pays a block-wide exchange per reduction); longer rows: a block per row
    // (with few rows a block per row is what spreads the work over the SMs)
    const char* wm = getenv("B200_ROW_WARP_MAX");
    const int64_t warp_max = wm ? atoll(wm) : 1024;
    const int T = (Nr <= 64 || (Nr <= warp_max && Nk >= 1184)) ? 32 : 256, per_block = 256 / T;
    // V consecutive elements of the row per thread and round, moved with 16-byte accesses where a tensor is read or
    // written at the row element's own position: 8 when the row's tensors include 2-byte types, else 4
    int V = 1;
    if (!getenv("B200_NO_WIDE_ROWS")) {
      bool two = false;
      for (Group* g : rc.stages)
        for (Op* mop : g->members) {
          two = two || dt_size(mop->results[0]->type.dt) == 2;
          for (Value* ov : mop->operands) two = two || (ov->type.numel() == Nk * Nr && dt_size(ov->type.dt) == 2);
        }
      if (two && Nr % 8 == 0) V = 8;
      else if (Nr % 4 == 0) V = 4;
    }
    const std::string it = "int";
    std::set<Op*> chain_members;
    for (Group* g : rc.stages) chain_members.insert(g->members.begin(), g->members.end());
    // a value needs memory when somebody outside the chain reads it (looking through the broadcasts and other
    // duplicable operations that are evaluated inline by their users)
    std::function<bool(Value*)> stored = [&](Value* v) -> bool {
      if (st.returned.count(v)) return true;
      for (Op* u : st.users[v]) {
        if (chain_members.count(u)) {
          // a cheap operation can be evaluated by several kernels: all of them must be stages of this chain
          bool all_inside = true;
          auto gi = st.group_of.find(u);
          if (gi != st.group_of.end())
            for (Group* ug : gi->second) all_inside = all_inside && std::find(rc.stages.begin(), rc.stages.end(), ug) != rc.stages.end();
          if (all_inside) continue;
          return true;
        }
        if (is_dup(u) && !st.dup_materialize.count(u) && !slot_of.count(u->results[0])) {
          if (stored(u->results[0])) return true;
          continue;
        }
        return true;
      }
      return false;
    };
    // kept index decomposition, shared by all stages
    Emitter pe;
    pe.is_internal = [](Op*) { return false; };
    pe.idx_t = it;
    pe.name_prefix = "k";
    pe.indent_ = 2;
    Ctx kc;
    kc.shape = rc.kept_shape;
    kc.lin = "o";
    pe.ensure_idx(kc);
    std::vector<Value*> ins, outs;
    std::ostringstream decl, body;
    std::set<Op*> members_so_far;
    std::map<Value*, std::string> bound;
    std::string label = "row{";
    int stage_no = 0;
    for (Group* g : rc.stages) {
      label += (stage_no ? " > " : "") + group_label(g);
      members_so_far.insert(g->members.begin(), g->members.end());
      Emitter em;
      em.idx_t = it;
      em.name_prefix = std::string(1, (char)('a' + stage_no));
      em.indent_ = 6;
      em.seed_inputs(ins);
      em.bound = bound;
      const std::set<Op*> ms = members_so_far;
      em.is_internal = [this, ms, &st](Op* o) {
        return (ms.count(o) && categorize(o) != Cat::REDUCE) || (is_dup(o) && !st.dup_materialize.count(o) && !slot_of.count(o->results[0]));
      };
      Ctx rctx;
      rctx.shape = rc.red_shape;
      rctx.lin = "r";
      em.ensure_idx(rctx);
      Ctx oc;
      oc.shape = rc.in_shape;
      oc.idx = kc.idx;
      oc.idx.insert(oc.idx.end(), rctx.idx.begin(), rctx.idx.end());
      oc.lin = "lin";
      // the loop over the row's elements around a stage's code; `stage_outs` are the (output number, value) pairs the
      // stage stores at the element's own position
      auto row_loop = [&](Emitter& e2, const std::vector<std::pair<size_t, Value*>>& stage_outs) -> std::string {
        std::string inner = e2.str();
        if (V == 1)
          return "    for (" + it + " r = lane; r < " + std::to_string(Nr) + "; r += " + std::to_string(T) + ") {\n      const " + it +
                 " lin = o * " + std::to_string(Nr) + " + r;\n" + inner + "    }\n";
        std::ostringstream pre, post;
        for (size_t k = 0; k < e2.inputs.size(); k++) {
          Value* in = e2.inputs[k];
          const int es = dt_size(in->type.dt);
          if (in->type.numel() != Nk * Nr || (es != 1 && es != 2 && es != 4) || (V * es) % 4 != 0) continue;
          const std::string nm = "in" + std::to_string(k);
          if (!replace_word(inner, nm + "[lin]", "v" + nm + "[e]")) continue;
          pre << "      __align__(16) " << s_type(in->type.dt) << " v" << nm << "[" << V << "];\n" << wide_move("v" + nm, nm, V, es, true, 6);
        }
        for (auto& so : stage_outs) {
          const int es = dt_size(so.second->type.dt);
          if ((es != 1 && es != 2 && es != 4) || (V * es) % 4 != 0) continue;
          const std::string nm = "out" + std::to_string(so.first);
          if (!replace_word(inner, nm + "[lin]", "v" + nm + "[e]")) continue;
          pre << "      __align__(16) " << s_type(so.second->type.dt) << " v" << nm << "[" << V << "];\n";
          post << wide_move("v" + nm, nm, V, es, false, 6);
        }
        return "    for (" + it + " rb = lane * " + std::to_string(V) + "; rb < " + std::to_string(Nr) + "; rb += " + std::to_string(T * V) +
               ") {\n      const " + it + " base = o * " + std::to_string(Nr) + " + rb;\n" + pre.str() +
               "      #pragma unroll\n      for (int e = 0; e < " + std::to_string(V) + "; ++e) {\n      const " + it + " r = rb + e;\n      const " +
               it + " lin = base + e;\n" + inner + "      }\n" + post.str() + "    }\n";
      };
      if (g->is_reduce) {
        std::vector<Value*> operands, results;
        std::vector<std::string> inits;
        std::vector<DT> dts;
        struct Part { Block* body; size_t n; };
        std::vector<Part> parts;
        for (Op* root : g->roots) {
          const size_t np = root->operands.size() / 2;
          for (size_t k = 0; k < np; k++) {
            operands.push_back(root->operands[k]);
            DenseValue dv = attr_dense(root->operands[np + k]->def->attr("value"));
            inits.push_back(literal(dv.type.dt, dv.data.data()));
            results.push_back(root->results[k]);
            dts.push_back(root->results[k]->type.dt);
          }
          parts.push_back({root->regions[0].get(), np});
        }
        const size_t n = operands.size();
        std::vector<std::string> vals;
        for (Value* v : operands) vals.push_back(em.emit(v, oc));
        em.round_small_floats = false;
        auto combine = [&](Emitter& e, const std::string& other, bool from_vals) {
          size_t base = 0;
          for (auto& part : parts) {
            std::vector<std::string> a;
            for (size_t k = 0; k < part.n; k++) a.push_back("acc" + std::to_string(base + k));
            for (size_t k = 0; k < part.n; k++) a.push_back(from_vals ? vals[base + k] : other + std::to_string(base + k));
            auto c = e.emit_scalar_region(part.body, a);
            for (size_t k = 0; k < part.n; k++) e.line("acc" + std::to_string(base + k) + " = " + c[k] + ";");
            base += part.n;
          }
        };
        combine(em, "", true);
        const std::string sn = std::to_string(stage_no);
        for (size_t k = 0; k < n; k++) {
          decl << "  " << c_type(dts[k]) << " S" << sn << "_" << k << ";\n";
          if (T == 256) decl << "  __shared__ " << c_type(dts[k]) << " sm" << sn << "_" << k << "[8];\n";
        }
        body << "  {\n";
        for (size_t k = 0; k < n; k++) body << "    " << c_type(dts[k]) << " acc" << k << " = " << inits[k] << ";\n";
        body << "    {\n" << row_loop(em, {}) << "    }\n";
        body << "    #pragma unroll\n    for (int m = 16; m >= 1; m >>= 1) {\n";
        for (size_t k = 0; k < n; k++) body << "      const " << c_type(dts[k]) << " oth" << k << " = shfl_xor(acc" << k << ", m);\n";
        {
          Emitter te;
          te.idx_t = it;
          te.name_prefix = em.name_prefix + "t";
          te.indent_ = 6;
          te.round_small_floats = false;
          combine(te, "oth", false);
          body << te.str();
        }
        body << "    }\n";
        if (T == 256) {
          body << "    if ((threadIdx.x & 31) == 0) {";
          for (size_t k = 0; k < n; k++) body << " sm" << sn << "_" << k << "[threadIdx.x >> 5] = acc" << k << ";";
          body << " }\n    __syncthreads();\n";
          for (size_t k = 0; k < n; k++) body << "    acc" << k << " = sm" << sn << "_" << k << "[0];\n";
          body << "    for (int w = 1; w < 8; ++w) {\n";
          for (size_t k = 0; k < n; k++) body << "      const " << c_type(dts[k]) << " oth" << k << " = sm" << sn << "_" << k << "[w];\n";
          Emitter te;
          te.idx_t = it;
          te.name_prefix = em.name_prefix + "u";
          te.indent_ = 6;
          te.round_small_floats = false;
          combine(te, "oth", false);
          body << te.str() << "    }\n";
        }
        for (size_t k = 0; k < n; k++) body << "    S" << sn << "_" << k << " = acc" << k << ";\n";
        body << "  }\n";
        for (size_t k = 0; k < n; k++) {
          bound[results[k]] = "S" + sn + "_" + std::to_string(k);
          if (stored(results[k])) {
            body << "  if (lane == 0 && live) out" << outs.size() << "[o] = " << store_expr(dts[k], "S" + sn + "_" + std::to_string(k)) << ";\n";
            outs.push_back(results[k]);
          }
        }
      } else if (g->roots[0]->results[0]->type.dims != rc.in_shape) {
        // arithmetic on the rows' own values (a mean turned into a reciprocal root): every thread computes it
        Emitter ke;
        ke.idx_t = it;
        ke.name_prefix = em.name_prefix + "k";
        ke.indent_ = 2;
        ke.seed_inputs(ins);
        ke.bound = bound;
        ke.is_internal = em.is_internal;
        Ctx kctx = kc;
        for (Op* root : g->roots) {
          Value* v = root->results[0];
          const std::string e = ke.emit(v, kctx);
          const std::string nm = "K" + std::to_string(stage_no) + "_" + std::to_string(bound.size());
          ke.line(std::string("const ") + c_type(v->type.dt) + " " + nm + " = " + e + ";");
          bound[v] = nm;
          if (stored(v)) {
            ke.line("if (lane == 0 && live) out" + std::to_string(outs.size()) + "[o] = " + store_expr(v->type.dt, nm) + ";");
            outs.push_back(v);
          }
        }
        body << ke.str();
        ins = ke.inputs;
        stage_no++;
        continue;
      } else {
        std::vector<std::pair<Value*, std::string>> stores;
        for (Op* root : g->roots)
          if (stored(root->results[0])) stores.push_back({root->results[0], em.emit(root->results[0], oc)});
        if (!stores.empty()) {
          std::vector<std::pair<size_t, Value*>> stage_outs;
          for (auto& sv : stores) {
            em.line("out" + std::to_string(outs.size()) + "[lin] = " + store_expr(sv.first->type.dt, sv.second) + ";");
            stage_outs.push_back({outs.size(), sv.first});
            outs.push_back(sv.first);
          }
          body << "  if (live) {\n" << row_loop(em, stage_outs) << "  }\n";
        }
      }
      ins = em.inputs;
      stage_no++;
    }
    label += "}";
    std::ostringstream src;
    src << "extern \"C\" __global__ void __launch_bounds__(256) @NAME@(" << signature(outs, ins) << ") {\n";
    // rows past the end (the last block of the warp-per-row form) work on the last row and store nothing
    src << "  const " << it << " o_raw = (" << it << ")blockIdx.x * " << per_block << " + threadIdx.x / " << T << ";\n";
    src << "  const bool live = o_raw < " << Nk << ";\n";
    src << "  const " << it << " o = live ? o_raw : " << Nk - 1 << ";\n";
    src << "  const int lane = threadIdx.x % " << T << ";\n";
    src << pe.str() << decl.str() << body.str() << "}\n";
    Launch L;
    L.kernel = add_kernel(src.str(), "row");
    L.grid[0] = (unsigned)((Nk + per_block - 1) / per_block); L.grid[1] = L.grid[2] = 1;
    L.block[0] = 256; L.block[1] = L.block[2] = 1;
    L.outs = outs;
    L.ins = ins;
    if (outs.empty()) return;
    add_launch(plan, L, label, st);
  }

  // A large transpose that moves the innermost dimension, standing alone (or several of them concatenated along
  // dimension 0, what the weights of a decode loop become): moved by the tiled kernel that stages 32 x 32 (64 x 64)
  // tiles through shared memory, so that reads and writes are both whole lines. The index-rewriting form inside a
  // fused kernel reads or writes with a stride. Input dims A ++ X ++ Y, output dims A ++ Y ++ X.
  bool lower_tiled_transpose(Group* g, Plan& plan, BlockState& st) {
    if (g->roots.size() != 1 || getenv("B200_NO_TILED_TRANSPOSE")) return false;
    Op* root = g->roots[0];
    Value* out = root->results[0];
    const size_t es = dt_size(out->type.dt);
    if ((es != 2 && es != 4) || out->type.numel() < (1 << 16)) return false;
    struct Part { Value* src; long long B, R, C, dst_off; };
    std::vector<Part> parts;
    auto canonical = [&](Op* t, Part& p) -> bool {
      if (t->short_name() != "transpose") return false;
      Value* src = t->operands[0];
      if (!slot_of.count(src) || (src->def && is_dup(src->def) && !st.dup_materialize.count(src->def))) return false;
      auto perm = attr_i64s(t->attr("permutation"));
      const int n = (int)perm.size();
      for (int a = 0; a < n - 1; a++) {
        bool ok = true;
        for (int i = 0; i < a && ok; i++) ok = perm[i] == i;
        if (!ok) break;
        for (int x = 1; a + x < n; x++) {
          const int y = n - a - x;
          bool match = true;
          for (int i = 0; i < y && match; i++) match = perm[a + i] == a + x + i;
          for (int i = 0; i < x && match; i++) match = perm[a + y + i] == a + i;
          if (!match) continue;
          p.src = src;
          p.B = p.R = p.C = 1;
          for (int i = 0; i < a; i++) p.B *= src->type.dims[i];
          for (int i = a; i < a + x; i++) p.R *= src->type.dims[i];
          for (int i = a + x; i < n; i++) p.C *= src->type.dims[i];
          return p.B <= 65535 && p.R > 1 && p.C > 1 && (es == 4 || (p.R % 2 == 0 && p.C % 2 == 0)) && (p.R + 31) / 32 <= 65535;
        }
      }
      return false;
    };
    long long dst_ld = 0, dst_bs = 0;
    if (g->members.size() == 1) {
      Part p;
      if (!canonical(root, p)) return false;
      p.dst_off = 0;
      dst_ld = p.R;
      dst_bs = p.R * p.C;
      parts.push_back(p);
    } else {
      // concatenate along dimension 0 of rank-2 transposes
      if (root->short_name() != "concatenate" || attr_int(root->attr("dimension")) != 0 || out->type.rank() != 2) return false;
      if (g->members.size() != root->operands.size() + 1) return false;
      long long off = 0;
      for (Value* o : root->operands) {
        Part p;
        if (!o->def || !g->members.count(o->def) || o->type.rank() != 2 || !canonical(o->def, p) || p.B != 1) return false;
        p.dst_off = off * out->type.dims[1];
        off += o->type.dims[0];
        parts.push_back(p);
      }
      dst_ld = out->type.dims[1];
      dst_bs = 0;
      for (auto& p : parts) if (p.R != dst_ld) return false;
    }
    ensure_slot(out, st);
    for (auto& p : parts) {
      Step s;
      s.kind = Step::TRANSPOSE;
      s.label = "tiled transpose";
      s.args = {slot_of.at(out), slot_of.at(p.src)};
      s.iparams = {(long long)es, p.B, p.R, p.C, dst_ld, dst_bs, p.dst_off};
      plan.steps.push_back(std::move(s));
    }
    return true;
  }

  void emit_group(Group* g, Plan& plan, BlockState& st) {
    if (!g->is_reduce) {
      // a lone reshape of a value that already lives in memory is a view
      if (g->members.size() == 1 && g->roots.size() == 1 && g->roots[0]->short_name() == "reshape") {
        Value* src = g->roots[0]->operands[0];
        if (slot_of.count(src) && !(src->def && is_dup(src->def) && !st.dup_materialize.count(src->def))) {
          slot_of[g->roots[0]->results[0]] = slot_of.at(src);
          return;
        }
      }
      if (g->roots[0]->results[0]->type.numel() == 0) {
        for (auto* r : g->roots) ensure_slot(r->results[0], st);
        return;
      }
      if (lower_tiled_transpose(g, plan, st)) return;
      if (g->roots.size() == 1 && window_updates.count(g->roots[0])) {
        Op* d = g->roots[0];
        slot_of[d->results[0]] = slot_of.at(d->operands[0]);
        Launch L = gen_window_update(g, st);
        add_launch(plan, L, group_label(g) + ".window", st);
        return;
      }
      Launch L = gen_pointwise(g, st);
      add_launch(plan, L, group_label(g), st);
      return;
    }
    // one part per reduce op of the group (sibling reductions over the same index space share the kernel)
    Op* r = g->roots[0];
    ReduceGen rg;
    rg.in_shape = r->operands[0]->type.dims;
    rg.dims = attr_i64s(r->attr("dimensions"));
    std::vector<Value*> outs;
    for (Op* root : g->roots) {
      const size_t np = root->operands.size() / 2;
      ReducePart part;
      part.operands.assign(root->operands.begin(), root->operands.begin() + np);
      part.inits.assign(root->operands.begin() + np, root->operands.end());
      part.body = root->regions[0].get();
      for (auto* v : root->results) part.dts.push_back(v->type.dt);
      for (auto* iv : part.inits)
        if (!(iv->def && iv->def->short_name() == "constant")) {
          if (!slot_of.count(iv)) throw CompileError("reduce: init value must be a constant or live in memory");
        }
      outs.insert(outs.end(), root->results.begin(), root->results.end());
      rg.parts.push_back(std::move(part));
    }
    std::vector<int64_t> kept_shape;
    int64_t Nk = 1, Nr = 1, trailing = 1;
    int last_red = -1;
    for (size_t d = 0; d < rg.in_shape.size(); d++) {
      bool red = std::find(rg.dims.begin(), rg.dims.end(), (int64_t)d) != rg.dims.end();
      if (red) { Nr *= rg.in_shape[d]; last_red = (int)d; }
      else { Nk *= rg.in_shape[d]; kept_shape.push_back(rg.in_shape[d]); }
    }
    for (size_t d = last_red + 1; d < rg.in_shape.size(); d++) trailing *= rg.in_shape[d];
    if (Nk == 0) { for (auto* o : outs) ensure_slot(o, st); return; }
    bool col = trailing >= 16;
    // parallelism: split the reduced range over blockIdx.y when there are few outputs
    // (the row strategy gives an output a whole block from 128 reduced elements on, a warp below)
    int64_t blocks = col ? (Nk + 31) / 32 : (Nr >= 128 ? Nk : (Nk + 7) / 8);
    // enough blocks to fill 148 SMs with 2048 threads each (1184 blocks of 256 threads), each split keeping
    // at least a few unrolled iterations per thread
    int64_t per_split_min = col ? 64 : (Nr >= 1024 ? 2048 : 256);
    const int64_t target_blocks = 1184;
    int splits = 1;
    if (blocks < target_blocks && Nr > per_split_min) {
      splits = (int)std::min<int64_t>((target_blocks + blocks - 1) / blocks, (Nr + per_split_min - 1) / per_split_min);
      splits = std::max(1, std::min(splits, 1024));
    }
    // a few thousand elements in all: a second launch costs more than the parallelism of a split returns
    if (Nk * Nr <= 32768) splits = 1;
    auto internal = [this, g, &st](Op* o) {
      return (g->members.count(o) && categorize(o) != Cat::REDUCE) || (is_dup(o) && !st.dup_materialize.count(o) && !slot_of.count(o->results[0]));
    };
    if (splits == 1) {
      Launch L = gen_reduce_kernel(rg, internal, 1, col, outs);
      add_launch(plan, L, group_label(g), st);
      return;
    }
    // pass 1 -> partials [splits, kept...]; pass 2 reduces dim 0 with the same combiners
    std::vector<Value*> partials;
    ReduceGen r2;
    for (auto& part : rg.parts) {
      ReducePart p2;
      for (size_t k = 0; k < part.operands.size(); k++) {
        TensorType t;
        t.dt = part.dts[k];
        t.dims.push_back(splits);
        for (auto s : kept_shape) t.dims.push_back(s);
        Value* pv = synth(t);
        partials.push_back(pv);
        p2.operands.push_back(pv);
      }
      p2.inits = part.inits;
      p2.body = part.body;
      p2.dts = part.dts;
      r2.parts.push_back(std::move(p2));
    }
    Launch L1 = gen_reduce_kernel(rg, internal, splits, col, partials);
    add_launch(plan, L1, group_label(g) + ".partial", st);
    r2.in_shape = partials[0]->type.dims;
    r2.dims = {0};
    // Pointwise kernels over the reduced shape whose inputs are all at hand once the sums exist (the per-channel
    // statistics, scale and shift of a batch norm, the gradient updates of its scale and bias) are evaluated by the
    // thread that holds the final sums instead of being launched on their own.
    std::vector<Group*> epi;
    std::string epi_label;
    if (opts.fuse && Nk <= 65536) {
      bool all_f32 = true;
      for (auto* o : outs) all_f32 = all_f32 && o->type.dt == DT::F32;
      std::set<Value*> at_hand(outs.begin(), outs.end());
      std::function<bool(Value*)> avail = [&](Value* v) -> bool {
        if (at_hand.count(v) || slot_of.count(v)) return true;
        Op* d = v->def;
        if (!d || d->parent != st.block) return false;
        if (is_dup(d) && !st.dup_materialize.count(d)) {
          for (auto* o : d->operands) if (!avail(o)) return false;
          return true;
        }
        return false;
      };
      bool grew = all_f32;
      while (grew && epi.size() < 6) {
        grew = false;
        for (auto& cand : st.groups) {
          Group* e = &cand;
          if (e->is_reduce || e->members.empty() || emitted.count(e) || absorbed.count(e) || e->members.size() > 48) continue;
          bool ok = true;
          for (Op* r : e->roots) ok = ok && r->results.size() == 1 && r->results[0]->type.dims == outs[0]->type.dims &&
                                       categorize(r) == Cat::ELEMENTWISE;
          bool uses_result = false;
          for (Op* m : e->members) {
            if (!ok) break;
            if (categorize(m) != Cat::ELEMENTWISE && !is_dup(m)) { ok = false; break; }
            for (Value* o : m->operands) {
              if (o->def && e->members.count(o->def)) continue;
              if (at_hand.count(o)) uses_result = true;
              if (!avail(o)) { ok = false; break; }
            }
          }
          if (!ok || !uses_result) continue;
          epi.push_back(e);
          absorbed.insert(e);
          for (Op* r : e->roots) at_hand.insert(r->results[0]);
          epi_label += "+" + group_label(e);
          grew = true;
          if (epi.size() >= 6) break;
        }
      }
    }
    // few outputs: one warp per output walks the partials (a column kernel would run as two or three blocks)
    Launch L2 = gen_reduce_kernel(r2, [](Op*) { return false; }, 1, Nk >= 2048, outs, &epi, &outs, &st);
    add_launch(plan, L2, group_label(g) + ".final" + epi_label, st);
  }

  void materialize_dup(Op* op, Plan& plan, BlockState& st) {
    Value* v = op->results[0];
    if (slot_of.count(v)) return;
    if (op->short_name() == "constant") {
      DenseValue dv = attr_dense(op->attr("value"));
      slot_of[v] = const_slot(dv.type, dv.data);
      return;
    }
    Group g;
    g.id = next_group_id++;
    g.members.insert(op);
    g.roots.push_back(op);
    g.identity.insert(op);
    if (v->type.numel() == 0) { ensure_slot(v, st); return; }
    // operand of a broadcast must itself be in memory or duplicable
    Launch L = gen_pointwise(&g, st);
    add_launch(plan, L, op->short_name(), st);
  }

  long long static_trip_count(Op* w) {
    // Counted-loop form (src/pjrt_plugin/ops/control_flow.cc:223-312): cond is `compare LT, counter, limit`
    // with a constant limit, body adds a positive constant to the counter, init is a constant.
    Block* cond = w->regions[0].get();
    Block* body = w->regions[1].get();
    Op* ret = cond->ops.back().get();
    if (ret->operands.size() != 1 || !ret->operands[0]->def) return -1;
    Op* cmp = ret->operands[0]->def;
    if (cmp->short_name() != "compare" || attr_enum(cmp->attr("comparison_direction")) != "LT") return -1;
    Value* counter = cmp->operands[0];
    if (counter->def || counter->owner != cond) return -1;
    int ci = counter->arg_index;
    auto const_int = [&](Value* v, long long& out) -> bool {
      if (!v->def || v->def->short_name() != "constant") return false;
      DenseValue dv = attr_dense(v->def->attr("value"));
      if (dv.type.numel() != 1 || !dt_is_int(dv.type.dt)) return false;
      long long x = 0;
      switch (dv.type.dt) {
        case DT::I32: { int32_t t; memcpy(&t, dv.data.data(), 4); x = t; break; }
        case DT::U32: { uint32_t t; memcpy(&t, dv.data.data(), 4); x = t; break; }
        case DT::I64: case DT::U64: { int64_t t; memcpy(&t, dv.data.data(), 8); x = t; break; }
        default: return false;
      }
      out = x;
      return true;
    };
    long long limit, init, step;
    if (!const_int(cmp->operands[1], limit)) return -1;
    if (!const_int(w->operands[ci], init)) return -1;
    Op* bret = body->ops.back().get();
    Value* next = bret->operands[ci];
    if (!next->def || next->def->short_name() != "add") return -1;
    Value *a = next->def->operands[0], *b = next->def->operands[1];
    Value* barg = body->args[ci];
    Value* other = a == barg ? b : (b == barg ? a : nullptr);
    if (!other || !const_int(other, step) || step <= 0) return -1;
    if (limit <= init) return 0;
    return (limit - init + step - 1) / step;
  }

  void plan_block(Block* block, Plan& plan, int arena, const std::vector<Value*>& returned_vals) {
    BlockState st;
    st.block = block;
    st.arena = arena;
    int pos = 0;
    for (auto& op : block->ops) {
      op->pos = pos++;
      st.ops.push_back(op.get());
    }
    for (auto* v : returned_vals) st.returned.insert(v);
    for (auto* op : st.ops) {
      if (categorize(op) == Cat::RETURN) continue;
      for (auto* o : op->operands) st.users[o].push_back(op);
      for (auto& r : op->regions) lift_uses(r.get(), op, block, st);
    }
    // dead code: results nobody reads (e.g. the input gradient of the first convolution) are not computed
    {
      std::set<Op*> live;
      for (int i = (int)st.ops.size() - 1; i >= 0; i--) {
        Op* op = st.ops[i];
        Cat c = categorize(op);
        bool keep = c == Cat::RETURN || c == Cat::ALL_REDUCE || c == Cat::ALL_GATHER;
        for (auto* r : op->results) {
          if (st.returned.count(r)) keep = true;
          for (auto* u : st.users[r])
            if (live.count(u)) keep = true;
        }
        if (keep) live.insert(op);
      }
      std::vector<Op*> kept;
      for (auto* op : st.ops)
        if (live.count(op)) kept.push_back(op);
      if (kept.size() != st.ops.size()) {
        st.ops = kept;
        st.users.clear();
        for (auto* op : st.ops) {
          if (categorize(op) == Cat::RETURN) continue;
          for (auto* o : op->operands) st.users[o].push_back(op);
          for (auto& r : op->regions) lift_uses(r.get(), op, block, st);
        }
      }
    }
    build_groups(st);
    for (auto& g : st.groups)
      for (auto* m : g.members) g.max_pos = std::max(g.max_pos, m->pos);
    if (opts.fuse) merge_sibling_reductions(st);

    // units and their dependencies
    std::vector<Unit> units;
    std::map<Op*, int> unit_of_op;          // unit that writes the op's results to memory
    std::map<Group*, int> unit_of_group;
    for (auto* op : st.ops) {
      Cat c = categorize(op);
      if (c == Cat::RETURN) continue;
      auto git = st.group_of.find(op);
      if (git != st.group_of.end()) {
        for (Group* g : git->second) {
          if (!unit_of_group.count(g)) {
            Unit u;
            u.kind = Unit::GROUP;
            u.group = g;
            u.prio = g->max_pos;
            unit_of_group[g] = (int)units.size();
            units.push_back(u);
          }
          if (std::find(g->roots.begin(), g->roots.end(), op) != g->roots.end()) unit_of_op[op] = unit_of_group[g];
        }
        continue;
      }
      if (c == Cat::DUP) {
        if (!st.dup_materialize.count(op)) continue;
        Unit u;
        u.kind = Unit::CONST_MAT;
        u.op = op;
        u.prio = op->pos;
        unit_of_op[op] = (int)units.size();
        units.push_back(u);
        continue;
      }
      Unit u;
      u.kind = Unit::OP;
      u.op = op;
      u.prio = op->pos;
      unit_of_op[op] = (int)units.size();
      units.push_back(u);
    }
    size_t U = units.size();
    std::vector<std::set<int>> succ(U);
    std::vector<int> indeg(U, 0);
    auto add_dep = [&](Value* v, int consumer) {
      // walks through duplicable ops that are evaluated inline
      std::vector<Value*> work{v};
      std::set<Value*> seen;
      while (!work.empty()) {
        Value* x = work.back();
        work.pop_back();
        if (!seen.insert(x).second) continue;
        Op* d = x->def;
        if (!d || d->parent != block) continue;
        auto it = unit_of_op.find(d);
        if (it != unit_of_op.end()) {
          if (it->second != consumer && succ[it->second].insert(consumer).second) indeg[consumer]++;
          continue;
        }
        if (is_dup(d)) for (auto* o : d->operands) work.push_back(o);
      }
    };
    std::function<void(Block*, int)> nested_deps = [&](Block* b, int consumer) {
      for (auto& op : b->ops) {
        for (auto* o : op->operands) add_dep(o, consumer);
        for (auto& r : op->regions) nested_deps(r.get(), consumer);
      }
    };
    for (auto* op : st.ops) {
      std::vector<int> consumers;
      auto git = st.group_of.find(op);
      if (git != st.group_of.end()) for (Group* g : git->second) consumers.push_back(unit_of_group.at(g));
      else {
        auto it = unit_of_op.find(op);
        if (it != unit_of_op.end()) consumers.push_back(it->second);
      }
      for (int cu : consumers) {
        for (auto* o : op->operands) add_dep(o, cu);
        for (auto& r : op->regions) nested_deps(r.get(), cu);
      }
    }
    // Kahn with original position as priority
    typedef std::pair<int, int> PI;
    std::priority_queue<PI, std::vector<PI>, std::greater<PI>> ready;
    for (size_t u = 0; u < U; u++)
      if (indeg[u] == 0) ready.push({units[u].prio, (int)u});
    std::vector<int> order;
    while (!ready.empty()) {
      int u = ready.top().second;
      ready.pop();
      order.push_back(u);
      for (int s : succ[u])
        if (--indeg[s] == 0) ready.push({units[s].prio, s});
    }
    if (order.size() != U) {
      std::string msg = "internal: fusion produced a cyclic schedule:";
      // find one cycle among the unscheduled units
      std::set<int> remaining;
      for (size_t u = 0; u < U; u++)
        if (std::find(order.begin(), order.end(), (int)u) == order.end()) remaining.insert((int)u);
      std::vector<int> path;
      std::set<int> on_path;
      int cur = *remaining.begin();
      while (!on_path.count(cur)) {
        on_path.insert(cur);
        path.push_back(cur);
        int nxt = -1;
        for (int p2 : remaining)
          if (succ[p2].count(cur)) { nxt = p2; break; }      // walk to an unscheduled predecessor
        if (nxt < 0) break;
        cur = nxt;
      }
      std::set<int> cyc;
      bool in = false;
      for (int u : path) { if (u == cur) in = true; if (in) cyc.insert(u); }
      int shown = 0;
      for (size_t u = 0; u < U && shown < 8; u++) {
        if (!cyc.count((int)u)) continue;
        shown++;
        msg += "\n  unit " + std::to_string(u) + " prio " + std::to_string(units[u].prio) + " ";
        if (units[u].kind == Unit::GROUP) {
          msg += group_label(units[u].group) + " members:";
          for (auto* m : units[u].group->members) msg += " " + m->short_name() + "@" + std::to_string(m->pos);
          msg += " roots:";
          for (auto* m : units[u].group->roots) msg += " " + m->short_name() + "@" + std::to_string(m->pos);
        } else msg += units[u].op->name + "@" + std::to_string(units[u].op->pos);
        msg += " -> succ:";
        for (int sx : succ[u]) msg += " " + std::to_string(sx);
      }
      throw CompileError(msg);
    }

    for (size_t oi = 0; oi < order.size(); oi++) {
      const int ui = order[oi];
      Unit& u = units[ui];
      if (u.kind == Unit::GROUP) {
        // a reduction over rows followed by kernels over the same rows: one launch for the chain
        RowChain rc;
        if (opts.fuse && !absorbed.count(u.group) && !getenv("B200_NO_ROW_FUSION") && row_form(u.group, rc)) {
          std::set<Op*> members;
          std::set<Value*> reduced, produced;
          auto take = [&](Group* g) {
            rc.stages.push_back(g);
            members.insert(g->members.begin(), g->members.end());
            const bool kept = g->is_reduce || g->roots[0]->results[0]->type.dims != rc.in_shape;
            for (Op* r : g->roots)
              for (Value* v : r->results) { produced.insert(v); if (kept) reduced.insert(v); }
          };
          if (row_safe(u.group, rc, u.group->members, reduced, st)) {
            take(u.group);
            // units that stand between the stages but read nothing of the chain (a constant, the scale vector of a
            // norm) go out in front of it
            std::vector<size_t> before;
            size_t last_stage = oi, n_before_at_last = 0;
            const bool dbg = getenv("B200_DEBUG_ROWS") != nullptr;
            for (size_t oj = oi + 1; oj < order.size() && oj < oi + 16 && rc.stages.size() < 8; oj++) {
              Unit& nu = units[order[oj]];
              if (nu.kind == Unit::CONST_MAT) {
                std::set<Value*> seen;
                std::function<bool(Value*)> dep = [&](Value* v) -> bool {
                  if (produced.count(v)) return true;
                  if (!seen.insert(v).second || !v->def || v->def->parent != block || !is_dup(v->def)) return false;
                  for (Value* o : v->def->operands) if (dep(o)) return true;
                  return false;
                };
                bool d = false;
                for (Value* o : nu.op->operands) d = d || dep(o);
                if (d) break;
                before.push_back(oj);
                continue;
              }
              if (nu.kind != Unit::GROUP || absorbed.count(nu.group) || nu.group->roots.empty()) {
                if (dbg) fprintf(stderr, "row chain stops: next unit is %s\n", nu.kind == Unit::GROUP ? "an absorbed or empty group" : nu.op->name.c_str());
                break;
              }
              Group* g = nu.group;
              if (g->roots.size() == 1 && window_updates.count(g->roots[0])) break;
              if (!reads_any(g, produced, st)) { before.push_back(oj); continue; }
              if (g->is_reduce) {
                RowChain r2;
                if (!row_form(g, r2) || r2.in_shape != rc.in_shape || r2.kept_shape != rc.kept_shape) {
                  if (dbg) fprintf(stderr, "row chain stops: %s has another row form\n", group_label(g).c_str());
                  break;
                }
              }
              std::set<Op*> m2 = members;
              m2.insert(g->members.begin(), g->members.end());
              if (!row_safe(g, rc, m2, reduced, st)) {
                if (dbg) fprintf(stderr, "row chain stops: %s is not row safe\n", group_label(g).c_str());
                break;
              }
              take(g);
              last_stage = oj;
              n_before_at_last = before.size();
            }
            if (rc.stages.size() >= 2) {
              before.resize(n_before_at_last);
              for (size_t ob : before) {
                Unit& bu = units[order[ob]];
                if (bu.kind == Unit::CONST_MAT) materialize_dup(bu.op, plan, st);
                else { emit_group(bu.group, plan, st); emitted.insert(bu.group); }
              }
              emit_row_chain(rc, plan, st);
              for (Group* g : rc.stages) emitted.insert(g);
              oi = last_stage;
              continue;
            }
          }
        }
        if (!absorbed.count(u.group)) emit_group(u.group, plan, st);
        emitted.insert(u.group);
        continue;
      }
      if (u.kind == Unit::CONST_MAT) { materialize_dup(u.op, plan, st); continue; }
      Op* op = u.op;
      Cat c = categorize(op);
      switch (c) {
        case Cat::CONV: case Cat::DOT: {
          ensure_slot(op->results[0], st);
          for (auto* o : op->operands)
            if (!slot_of.count(o)) throw CompileError("internal: operand of " + op->name + " has no storage");
          if (op->results[0]->type.numel() == 0) break;
          Dot16 native;
          if (c == Cat::DOT && dot16_geometry(op, native)) { lower_dot16(op, native, plan, st); break; }
          Step s = c == Cat::CONV ? lower_conv(op, st) : lower_dot(op, st);
          plan.steps.push_back(std::move(s));
          break;
        }
        case Cat::ALL_REDUCE: {
          // only sum over all partitions is implemented
          Block* body = op->regions[0].get();
          bool is_sum = body->ops.size() == 2 && body->ops[0]->short_name() == "add";
          if (!is_sum) throw CompileError("all_reduce: only a sum reduction is supported");
          if (op->has("replica_groups")) {
            DenseValue rg = attr_dense(op->attr("replica_groups"));
            if (rg.type.rank() != 2) throw CompileError("all_reduce: replica_groups must be rank 2");   // collectives.cc:22-33
            int64_t groups = rg.type.dims[0], gsize = rg.type.dims[1];
            if (groups > 1 || (gsize != opts.num_partitions && gsize != 0 && !(gsize == 1 && opts.num_partitions == 1)))
              throw CompileError("all_reduce: only one group spanning all " + std::to_string(opts.num_partitions) +
                                 " partitions is supported (got " + std::to_string(groups) + " x " + std::to_string(gsize) + ")");
          }
          for (size_t k = 0; k < op->operands.size(); k++) {
            Step s;
            s.kind = Step::ALL_REDUCE;
            s.label = op->name;
            s.dtype = op->operands[k]->type.dt;
            s.bytes = op->operands[k]->type.bytes();
            ensure_slot(op->results[k], st);
            s.args = {slot_of.at(op->operands[k]), slot_of.at(op->results[k])};
            plan.steps.push_back(std::move(s));
          }
          break;
        }
        case Cat::ALL_GATHER: {
          // every partition contributes its operand; the result concatenates them along all_gather_dim in partition
          // order (one group spanning all partitions, as for all_reduce). The reference has no collective beyond
          // src/pjrt_plugin/ops/collectives.cc:20-78; a shard_map program over N devices needs this one too.
          const int64_t dim = attr_int(op->attr("all_gather_dim"));
          if (op->has("replica_groups")) {
            DenseValue rg = attr_dense(op->attr("replica_groups"));
            if (rg.type.rank() != 2) throw CompileError("all_gather: replica_groups must be rank 2");
            int64_t groups = rg.type.dims[0], gsize = rg.type.dims[1];
            if (groups > 1 || (gsize != opts.num_partitions && gsize != 0 && !(gsize == 1 && opts.num_partitions == 1)))
              throw CompileError("all_gather: only one group spanning all " + std::to_string(opts.num_partitions) + " partitions is supported");
          }
          for (size_t k = 0; k < op->operands.size(); k++) {
            Value *in = op->operands[k], *out = op->results[k];
            if (dim < 0 || dim >= in->type.rank() || out->type.dims[dim] != in->type.dims[dim] * opts.num_partitions)
              throw CompileError("all_gather: result extent along all_gather_dim must be " + std::to_string(opts.num_partitions) + " times the operand's");
            ensure_slot(out, st);
            if (in->type.numel() == 0) continue;
            Step s;
            s.kind = Step::ALL_GATHER;
            s.label = op->name;
            s.dtype = in->type.dt;
            s.bytes = in->type.bytes();
            int64_t outer = 1;
            for (int64_t d = 0; d < dim; d++) outer *= in->type.dims[d];
            s.iparams = {outer, (long long)(in->type.bytes() / std::max<int64_t>(outer, 1))};    // rows, bytes per row of the operand
            s.args = {slot_of.at(in), slot_of.at(out)};
            if (outer > 1 && opts.num_partitions > 1) s.args.push_back(new_slot(Slot::TEMP, out->type, st.arena));   // [partition][operand]
            plan.steps.push_back(std::move(s));
          }
          break;
        }
        case Cat::WHILE: {
          Step s;
          s.kind = Step::WHILE;
          s.label = op->name;
          s.trip_count = static_trip_count(op);
          Block* cond = op->regions[0].get();
          Block* body = op->regions[1].get();
          size_t n = op->operands.size();
          for (size_t k = 0; k < n; k++) {
            ensure_slot(op->results[k], st);
            int sl = slot_of.at(op->results[k]);
            s.state.push_back(sl);
            s.init.push_back(slot_of.at(op->operands[k]));
            slot_of[cond->args[k]] = sl;
            slot_of[body->args[k]] = sl;
          }
          int a_cond = (int)prog.arena_bytes.size();
          prog.arena_bytes.push_back(0);
          int a_body = (int)prog.arena_bytes.size();
          prog.arena_bytes.push_back(0);
          auto pc = std::make_unique<Plan>();
          auto pb = std::make_unique<Plan>();
          Op* cret = cond->ops.back().get();
          Op* bret = body->ops.back().get();
          pc->arena = a_cond;
          pb->arena = a_body;
          plan_block(cond, *pc, a_cond, cret->operands);
          for (size_t k = 0; k < n; k++) {
            // state k is only ever updated in a window and handed back at position k: update it in place
            Value* r = bret->operands[k];
            Op* d = r->def;
            if (!d || d->parent != body || d->short_name() != "dynamic_update_slice" || d->operands[0] != body->args[k]) continue;
            std::function<int(Block*, Value*)> uses = [&](Block* blk, Value* v) {
              int c = 0;
              for (auto& o : blk->ops) {
                c += (int)std::count(o->operands.begin(), o->operands.end(), v);
                for (auto& reg : o->regions) c += uses(reg.get(), v);
              }
              return c;
            };
            // the old tensor has no other reader; the new one shares the state's memory, so whoever else reads it
            // (the attention product reading an updated key cache) finds it there
            if (uses(body, body->args[k]) != 1) continue;
            if (r->type.dims.empty() || r->type.numel() == 0 || getenv("B200_NO_WINDOW_UPDATE")) continue;
            window_updates.insert(d);
          }
          plan_block(body, *pb, a_body, bret->operands);
          s.pred = slot_of.at(cret->operands[0]);
          persistent.insert(s.pred);
          std::set<int> state_set(s.state.begin(), s.state.end());
          for (size_t k = 0; k < n; k++) {
            int ns = slot_of.at(bret->operands[k]);
            if (ns != s.state[k] && state_set.count(ns)) {
              // a carried value handed to another position: stage it so the copies below cannot clobber it
              int tmp = new_slot(Slot::TEMP, prog.slots[ns].type, a_body);
              Step c;
              c.kind = Step::MEMCPY;
              c.label = "loop-carried permutation";
              c.args = {tmp, ns};
              c.bytes = prog.slots[ns].type.bytes();
              pb->steps.push_back(std::move(c));
              ns = tmp;
            }
            persistent.insert(ns);
            s.next.push_back(ns);
          }
          // A carried value whose next value is a temporary of the body written once per iteration needs no copy:
          // the runtime exchanges the two pointers after each iteration. The body temporary then holds the state
          // during the following iteration, so it owns its memory for the whole body.
          s.swap.assign(n, 0);
          for (size_t k = 0; k < n; k++) {
            const int ns = s.next[k];
            const Slot& sn = prog.slots[ns];
            if (ns == s.state[k] || sn.kind != Slot::TEMP || sn.arena != a_body) continue;
            if (sn.bytes != prog.slots[s.state[k]].bytes || sn.bytes == 0) continue;
            if (std::count(s.next.begin(), s.next.end(), ns) != 1) continue;
            s.swap[k] = 1;
            whole_plan.insert(ns);
          }
          s.sub.push_back(std::move(pc));
          s.sub.push_back(std::move(pb));
          // every slot read inside the loop stays live across it: list them as args
          std::set<int> used;
          std::function<void(const Plan&)> collect = [&](const Plan& p) {
            for (auto& q : p.steps) {
              for (int a : q.args) used.insert(a);
              for (int a : q.init) used.insert(a);
              for (auto& sp : q.sub) collect(*sp);
            }
          };
          collect(*s.sub[0]);
          collect(*s.sub[1]);
          for (int a : used)
            if (prog.slots[a].arena == arena && prog.slots[a].kind == Slot::TEMP) s.args.push_back(a);
          plan.steps.push_back(std::move(s));
          break;
        }
        case Cat::CASE: {
          // lax.cond / lax.switch: the index is read back by the host, the chosen branch's plan runs and its
          // results are copied into the op's result slots (src/pjrt_plugin/ops/control_flow.cc:702-1317;
          // an index outside [0, branches) selects the last branch)
          Step s;
          s.kind = Step::CASE;
          s.label = op->name;
          s.pred = slot_of.at(op->operands[0]);
          for (auto* r : op->results) {
            ensure_slot(r, st);
            s.state.push_back(slot_of.at(r));
          }
          for (auto& reg : op->regions) {
            int a_br = (int)prog.arena_bytes.size();
            prog.arena_bytes.push_back(0);
            auto pb = std::make_unique<Plan>();
            pb->arena = a_br;
            Op* ret = reg->ops.back().get();
            plan_block(reg.get(), *pb, a_br, ret->operands);
            for (size_t k = 0; k < op->results.size(); k++) {
              int src = slot_of.at(ret->operands[k]);
              persistent.insert(src);
              Step c;
              c.kind = Step::MEMCPY;
              c.label = "case result";
              c.args = {s.state[k], src};
              c.bytes = prog.slots[src].type.bytes();
              pb->steps.push_back(std::move(c));
            }
            s.sub.push_back(std::move(pb));
          }
          std::set<int> used;
          std::function<void(const Plan&)> collect = [&](const Plan& p) {
            for (auto& q : p.steps) {
              for (int a : q.args) used.insert(a);
              for (int a : q.init) used.insert(a);
              for (auto& sp : q.sub) collect(*sp);
            }
          };
          for (auto& sp : s.sub) collect(*sp);
          s.args.push_back(s.pred);
          for (int a : used)
            if (prog.slots[a].arena == arena && prog.slots[a].kind == Slot::TEMP) s.args.push_back(a);
          plan.steps.push_back(std::move(s));
          break;
        }
        case Cat::SCATTER: {
          plan.steps.push_back(lower_scatter(op, plan, st));
          break;
        }
        case Cat::WINDOW: {
          Launch L = op->short_name() == "reduce_window" ? gen_reduce_window(op, st) : gen_select_and_scatter(op, st);
          add_launch(plan, L, op->short_name(), st);
          break;
        }
        case Cat::SORT: {
          lower_sort(op, plan, st);
          break;
        }
        case Cat::RNG: {
          lower_rng_bit_generator(op, plan, st);
          break;
        }
        case Cat::ATTENTION: {
          lower_decode_attention(op, plan, st);
          break;
        }
        case Cat::LINALG: {
          if (op->short_name() == "cholesky") lower_cholesky(op, plan, st);
          else lower_triangular_solve(op, plan, st);
          break;
        }
        case Cat::TOKEN: {
          ensure_slot(op->results[0], st);
          break;
        }
        case Cat::PARTITION_ID: {
          std::vector<uint8_t> b(4);
          uint32_t id = op->short_name() == "partition_id" ? (uint32_t)partition_id : 0u;
          memcpy(b.data(), &id, 4);
          slot_of[op->results[0]] = const_slot(op->results[0]->type, b);
          break;
        }
        default:
          throw CompileError("operation " + op->name + " is not supported by the B200 plugin");
      }
    }
    // block results must live in memory
    for (auto* v : returned_vals) {
      if (slot_of.count(v)) continue;
      if (v->def && v->def->parent == block && is_dup(v->def)) { materialize_dup(v->def, plan, st); continue; }
      throw CompileError("internal: returned value without storage: " + v->name);
    }
    bundle_independent_kernels(plan);
  }

  // ---- bundling of independent pointwise kernels --------------------------------------
  // Adjacent pointwise launches that do not depend on one another (the window updates of a scan body, the
  // accumulations at its end, optimizer updates of small parameters) become one launch: the bundle's grid is the
  // concatenation of the parts' grids and each block runs the part its index falls into. The parts keep their code
  // unchanged as device functions. Latency-bound plans pay per launch, so this is where their time goes.
  struct BundlePart { int kernel; unsigned grid; };

  int bundle_kernel(const std::vector<BundlePart>& parts) {
    std::ostringstream fns, sig, body;
    std::map<int, std::string> fn_of;
    int pi = 0;
    unsigned first = 0;
    body << "  unsigned bid = blockIdx.x;\n";
    for (size_t k = 0; k < parts.size(); k++) {
      const std::string& text = kernel_text[parts[k].kernel];
      const size_t name_at = text.find("@NAME@(");
      const size_t sig_end = text.find(") {\n", name_at);
      if (name_at == std::string::npos || sig_end == std::string::npos) return -1;
      const std::string params = text.substr(name_at + 7, sig_end - name_at - 7);
      if (!fn_of.count(parts[k].kernel)) {
        std::string fn = "@NAME@_p" + std::to_string(fn_of.size());
        std::string rest = text.substr(sig_end);          // ") {\n body }"
        for (auto p = rest.find("blockIdx.x"); p != std::string::npos; p = rest.find("blockIdx.x", p)) rest.replace(p, 10, "bid");
        fns << "static __device__ __forceinline__ void " << fn << "(const unsigned bid, " << params << rest << "\n";
        fn_of[parts[k].kernel] = fn;
      }
      // parameter types of the part, renamed for the bundle's own signature
      std::vector<std::string> names;
      size_t at = 0;
      while (at < params.size()) {
        size_t comma = params.find(", ", at);
        std::string one = params.substr(at, comma == std::string::npos ? std::string::npos : comma - at);
        size_t sp = one.find_last_of(' ');
        if (sp == std::string::npos) return -1;
        std::string nm = "a" + std::to_string(pi++);
        sig << (names.empty() && k == 0 ? "" : ", ") << one.substr(0, sp + 1) << nm;
        names.push_back(nm);
        if (comma == std::string::npos) break;
        at = comma + 2;
      }
      body << "  if (bid < " << first + parts[k].grid << "u) { " << fn_of[parts[k].kernel] << "(bid - " << first << "u";
      for (auto& nm : names) body << ", " << nm;
      body << "); return; }\n";
      first += parts[k].grid;
    }
    std::ostringstream src;
    src << fns.str() << "extern \"C\" __global__ void __launch_bounds__(" << kThreads << ") @NAME@(" << sig.str() << ") {\n"
        << body.str() << "}\n";
    return add_kernel(src.str(), "bundle");
  }

  void bundle_independent_kernels(Plan& plan) {
    if (getenv("B200_NO_BUNDLES")) return;
    auto eligible = [&](const Step& s) {
      return s.kind == Step::KERNEL && s.block[0] == (unsigned)kThreads && s.block[1] == 1 && s.block[2] == 1 && s.grid[1] == 1 &&
             s.grid[2] == 1 && s.n_outs > 0 && prog.kernels[s.kernel].name.rfind("fused_", 0) == 0;
    };
    std::vector<Step> out;
    size_t i = 0;
    while (i < plan.steps.size()) {
      if (!eligible(plan.steps[i])) { out.push_back(std::move(plan.steps[i++])); continue; }
      std::set<int> written, read;
      size_t j = i, nargs = 0;
      unsigned blocks = 0;
      for (; j < plan.steps.size() && j - i < 16; j++) {
        const Step& s = plan.steps[j];
        if (!eligible(s) || nargs + s.args.size() > 256 || (uint64_t)blocks + s.grid[0] > (1u << 30)) break;
        bool clash = false;
        for (size_t a = 0; a < s.args.size(); a++) {
          const bool w = (int)a < s.n_outs;
          if (written.count(s.args[a]) || (w && read.count(s.args[a]))) clash = true;
        }
        if (clash) break;
        for (size_t a = 0; a < s.args.size(); a++) ((int)a < s.n_outs ? written : read).insert(s.args[a]);
        nargs += s.args.size();
        blocks += s.grid[0];
      }
      int id = -1;
      if (j - i >= 2) {
        std::vector<BundlePart> parts;
        for (size_t k = i; k < j; k++) parts.push_back({plan.steps[k].kernel, plan.steps[k].grid[0]});
        id = bundle_kernel(parts);
      }
      if (id < 0) { out.push_back(std::move(plan.steps[i++])); continue; }
      Step b;
      b.kind = Step::KERNEL;
      b.kernel = id;
      b.grid[0] = blocks;
      b.block[0] = kThreads;
      b.n_outs = 0;                    // outputs and inputs interleave per part; bundles are not bundled again
      for (size_t k = i; k < j; k++) {
        b.label += (k > i ? " + " : "") + plan.steps[k].label;
        b.args.insert(b.args.end(), plan.steps[k].args.begin(), plan.steps[k].args.end());
      }
      out.push_back(std::move(b));
      i = j;
    }
    plan.steps = std::move(out);
  }

  // ---- overlap of gradient all-reduces with the backward pass ---------------------------
  // The all-reduces of a data-parallel step stand at the end of the program, after the last gradient. The
  // gradients of the late layers exist long before that: the run is cut into buckets of consecutive leaves (from
  // the last leaf backwards: most of the bytes first, a small bucket last), and every bucket moves up to just behind the last step
  // that touches one of its inputs. Moved or not, the buckets are issued on the collective stream; a JOIN step at
  // the run's old position makes the compute stream wait for them.
  void hoist_all_reduce_buckets(Plan& plan) {
    // On unless B200_NO_ALL_REDUCE_OVERLAP is set. Measured with the ResNet18 step on 2 / 4 / 8 B200s: 4.86 / 4.87 /
    // 4.97 ms per step against 4.89 / 4.92 / 5.03 ms with one all-reduce after the last gradient (with four equal
    // buckets, whose last one holds a quarter of the bytes and hides behind nothing, it was a loss).
    if (opts.num_partitions <= 1 || getenv("B200_NO_ALL_REDUCE_OVERLAP")) return;
    const size_t S = plan.steps.size();
    size_t b = 0;
    while (b < S && plan.steps[b].kind != Step::ALL_REDUCE) b++;
    if (b == S) return;
    size_t e = b;
    while (e + 1 < S && plan.steps[e + 1].kind == Step::ALL_REDUCE) e++;
    for (size_t i = e + 1; i < S; i++)
      if (plan.steps[i].kind == Step::ALL_REDUCE) return;          // several runs: leave the plan as it is
    const size_t n = e - b + 1;
    std::function<bool(const Step&, int)> mentions = [&](const Step& q, int slot) {
      for (auto* v : {&q.args, &q.state, &q.init, &q.next, &q.results})
        if (std::find(v->begin(), v->end(), slot) != v->end()) return true;
      if (q.pred == slot) return true;
      for (auto& sp : q.sub)
        for (auto& qq : sp->steps)
          if (mentions(qq, slot)) return true;
      return false;
    };
    std::vector<long long> ready(n, 0);      // index of the step behind which leaf k may be issued
    size_t total = 0;
    for (size_t k = 0; k < n; k++) {
      const int in = plan.steps[b + k].args[0];
      total += plan.steps[b + k].bytes;
      for (size_t i = b; i-- > 0;)
        if (mentions(plan.steps[i], in)) { ready[k] = (long long)i + 1; break; }
    }
    // buckets from the last leaf backwards
    struct Bucket { size_t lo, hi; long long at; };
    std::vector<Bucket> buckets;
    size_t hi = n, bytes = 0;
    long long at = 0;
    // Cut points in cumulative bytes from the last leaf: by default one, at 98 %: the late layers, whose gradients come
    // first and are nearly all of the bytes, go out as soon as they exist; a small last bucket follows the last
    // gradient, because what is produced last cannot hide behind anything. B200_ALL_REDUCE_CUTS="p1,p2,..." (per cent)
    // replaces the cut points (70, 97.5 measured 4.99 ms on 8 GPUs against 4.97 with the single cut).
    std::vector<double> cuts = {0.98};
    if (const char* cs = getenv("B200_ALL_REDUCE_CUTS")) {
      cuts.clear();
      for (const char* q = cs; *q;) {
        char* endp = nullptr;
        const double v = strtod(q, &endp);
        if (endp == q) break;
        cuts.push_back(v / 100.0);
        q = *endp == ',' ? endp + 1 : endp;
      }
    }
    size_t next_cut = 0, cum = 0;
    for (size_t k = n; k-- > 0;) {
      bytes += plan.steps[b + k].bytes;
      cum += plan.steps[b + k].bytes;
      at = std::max(at, ready[k]);
      const bool cut_here = next_cut < cuts.size() && (double)cum >= cuts[next_cut] * (double)total;
      if (cut_here || k == 0) {
        while (next_cut < cuts.size() && (double)cum >= cuts[next_cut] * (double)total) next_cut++;
        buckets.push_back({k, hi, at});
        hi = k;
        bytes = 0;
        at = 0;
      }
    }
    std::vector<Step> out;
    std::vector<Step> run;
    for (size_t k = 0; k < n; k++) {
      run.push_back(std::move(plan.steps[b + k]));
      run.back().overlapped = true;
    }
    auto emit_buckets_at = [&](long long pos, bool rest) {
      for (auto& bk : buckets) {
        const bool early = (long long)b - bk.at >= 8;            // enough work left behind it to hide anything
        if (rest ? early : (!early || bk.at != pos)) continue;
        for (size_t k = bk.lo; k < bk.hi; k++) out.push_back(std::move(run[k]));
      }
    };
    for (size_t i = 0; i < b; i++) {
      emit_buckets_at((long long)i, false);
      out.push_back(std::move(plan.steps[i]));
    }
    emit_buckets_at((long long)b, false);
    // buckets that are not worth moving stay here, in leaf order (one run)
    std::sort(buckets.begin(), buckets.end(), [](const Bucket& x, const Bucket& y) { return x.lo < y.lo; });
    emit_buckets_at(0, true);
    Step j;
    j.kind = Step::JOIN;
    j.label = "join collective stream";
    out.push_back(std::move(j));
    for (size_t i = e + 1; i < S; i++) out.push_back(std::move(plan.steps[i]));
    plan.steps = std::move(out);
  }

  int partition_id = 0;

  // ---- arena layout ---------------------------------------------------------------
  void layout_arena(Plan& plan) {
    const int arena = plan.arena;
    // liveness over the step sequence of this plan
    size_t S = plan.steps.size();
    std::map<int, std::pair<int, int>> live;    // slot -> [first, last]
    auto touch = [&](int slot, int at) {
      if (slot < 0) return;
      const Slot& s = prog.slots[slot];
      if (s.kind != Slot::TEMP || s.arena != arena) return;
      auto it = live.find(slot);
      if (it == live.end()) live[slot] = {at, at};
      else it->second.second = std::max(it->second.second, at);
    };
    for (size_t i = 0; i < S; i++) {
      Step& s = plan.steps[i];
      if (s.kind == Step::ALL_REDUCE) {
        // a run of all-reduces is issued as one NCCL group whose members execute concurrently: every operand
        // of the run is live over the whole run, so no output can reuse the memory of another member's input
        size_t b = i, e = i;
        while (b > 0 && plan.steps[b - 1].kind == Step::ALL_REDUCE) b--;
        while (e + 1 < S && plan.steps[e + 1].kind == Step::ALL_REDUCE) e++;
        for (int a : s.args) { touch(a, (int)b); touch(a, (int)e); }
        if (s.overlapped)
          for (size_t j = i + 1; j < S; j++)
            if (plan.steps[j].kind == Step::JOIN) {
              // issued on the collective stream: nothing may reuse the operands before the compute stream has joined
              for (int a : s.args) touch(a, (int)j);
              break;
            }
        continue;
      }
      for (int a : s.args) touch(a, (int)i);
      for (int a : s.state) touch(a, (int)i);
      for (int a : s.init) touch(a, (int)i);
      for (int a : s.results) touch(a, (int)i);
      touch(s.pred, (int)i);
    }
    // slots marked persistent (results of nested blocks) live to the end
    for (int ps : persistent)
      if (live.count(ps)) live[ps].second = (int)S;
    for (int ps : whole_plan)
      if (live.count(ps)) live[ps] = {0, (int)S};
    for (auto& sub_steps : plan.steps)
      for (auto& sp : sub_steps.sub) layout_arena(*sp);
    // The operands of a run of all-reduces (the gradient leaves of a data-parallel step) are laid out back to back,
    // inputs in one block and outputs in another, so that the runtime can reduce the whole run with one call over
    // one flat buffer instead of one operation per leaf. A pack is placed as a single block that lives from the
    // first member's first use to the last member's last use.
    std::map<int, std::vector<int>> packs;    // leader slot -> members in order (leader first)
    std::set<int> packed;
    for (size_t i = 0; i < S;) {
      if (plan.steps[i].kind != Step::ALL_REDUCE) { i++; continue; }
      size_t e = i;
      while (e + 1 < S && plan.steps[e + 1].kind == Step::ALL_REDUCE) e++;
      std::vector<int> ins, outs;
      bool ok = e > i;
      std::set<int> seen;
      for (size_t k = i; k <= e && ok; k++) {
        const Step& q = plan.steps[k];
        ok = q.dtype == plan.steps[i].dtype && q.bytes > 0;
        for (int a : q.args) ok = ok && live.count(a) && !packed.count(a) && seen.insert(a).second && !whole_plan.count(a);
        ins.push_back(q.args[0]);
        outs.push_back(q.args[1]);
      }
      if (ok && !getenv("B200_NO_FLAT_ALL_REDUCE")) {
        for (auto* v : {&ins, &outs}) {
          packs[(*v)[0]] = *v;
          for (int a : *v) {
            packed.insert(a);
            live[(*v)[0]].first = std::min(live[(*v)[0]].first, live[a].first);
            live[(*v)[0]].second = std::max(live[(*v)[0]].second, live[a].second);
          }
        }
      }
      i = e + 1;
    }
    // greedy first-fit by start time
    std::vector<std::pair<int, int>> order;   // (first, slot)
    for (auto& kv : live)
      if (!packed.count(kv.first) || packs.count(kv.first)) order.push_back({kv.second.first, kv.first});
    std::sort(order.begin(), order.end());
    struct Blk { size_t off, size; int last; };
    std::vector<Blk> active;
    size_t peak = 0;
    const bool no_reuse = getenv("B200_DEBUG_NO_REUSE") != nullptr;   // debugging: every temporary gets its own memory
    if (no_reuse)
      for (auto& pr : order) live[pr.second].second = 1 << 30;
    for (auto& pr : order) {
      int slot = pr.second;
      int first = pr.first, last = live[slot].second;
      size_t need = (prog.slots[slot].bytes + 255) & ~(size_t)255;
      auto pk = packs.find(slot);
      if (pk != packs.end()) {
        need = 0;
        for (int m : pk->second) need += (prog.slots[m].bytes + 255) & ~(size_t)255;
      }
      // drop blocks that ended before `first`
      active.erase(std::remove_if(active.begin(), active.end(), [&](const Blk& b) { return b.last < first; }), active.end());
      std::sort(active.begin(), active.end(), [](const Blk& a, const Blk& b) { return a.off < b.off; });
      size_t off = 0;
      for (auto& b : active) {
        if (off + need <= b.off) break;
        off = std::max(off, b.off + b.size);
      }
      prog.slots[slot].offset = off;
      if (pk != packs.end()) {
        size_t at = off;
        for (int m : pk->second) {
          prog.slots[m].offset = at;
          at += (prog.slots[m].bytes + 255) & ~(size_t)255;
        }
      }
      active.push_back({off, need, last});
      peak = std::max(peak, off + need);
    }
    prog.arena_bytes[arena] = std::max(prog.arena_bytes[arena], peak);
  }

  std::set<int> persistent;
  std::map<Op*, int> dup_depth;       // cheap operations evaluated in several kernels: links of duplicated users above them
  std::set<Op*> window_updates;       // dynamic_update_slice ops of loop bodies that update their loop state in place
  std::set<int> whole_plan;           // slots that own their memory for their whole plan (exchanged loop state)
  std::set<Group*> absorbed, emitted;     // pointwise groups folded into a reduction's second pass / groups already planned
};

void dump_plan(const CompiledProgram& prog, const Plan& p, std::ostringstream& os, int indent) {
  for (auto& s : p.steps) {
    os << std::string(indent, ' ');
    switch (s.kind) {
      case Step::KERNEL:
        os << "kernel " << prog.kernels[s.kernel].name << " grid=" << s.grid[0] << "x" << s.grid[1] << " block=" << s.block[0]
           << "x" << s.block[1] << " " << s.label;
        break;
      case Step::IGEMM:
        os << "igemm M=" << s.ig.M << " N=" << s.ig.N << " K=" << s.ig.K << " G=" << s.ig.groups << " splitK=" << s.ig.split_k
           << " a_contig=" << s.ig.a_contig << " b_contig=" << s.ig.b_contig << " vec=" << s.ig.vec << " seg=" << s.ig.seg << (s.ig.kt_stride ? " ktlist" : "") << (s.ig.a_tma ? " tmaA" : "") << " " << s.label;
        break;
      case Step::MEMCPY: os << "memcpy " << s.bytes; break;
      case Step::GEMM16:
        os << (s.g16.path == 0 ? "gemm16" : s.g16.path == 1 ? "gemv16_nc" : s.g16.path == 3 ? "gemv16_nc_small" : "gemv16_kc") << " M=" << s.g16.M << " N=" << s.g16.N
           << " K=" << s.g16.K << " G=" << s.g16.G << " a_kcontig=" << (s.g16.a_ks == 1) << " b_kcontig=" << (s.g16.b_ks == 1)
           << " bn=" << s.g16.bn << " splitK=" << s.g16.split_k << (s.g16.b_static ? " staticB" : "") << " out=" << (s.g16.c_kind == 2 ? "f32" : "16") << " " << s.label;
        break;
      case Step::TRANSPOSE:
        os << "transpose batch=" << s.iparams[1] << " rows=" << s.iparams[2] << " cols=" << s.iparams[3] << " bytes=" << s.iparams[0]
           << " dst_off=" << s.iparams[6];
        break;
      case Step::REPACK16: os << "repack16 rows=" << s.iparams[0] << " cols=" << s.iparams[1] << " ld " << s.iparams[3] << "->" << s.iparams[2]; break;
      case Step::WHILE:
        os << "while trip=" << s.trip_count << " exchanged=" << std::count(s.swap.begin(), s.swap.end(), (char)1) << "/" << s.state.size();
        break;
      case Step::CASE: os << "case branches=" << s.sub.size(); break;
      case Step::SCATTER: os << "scatter rows=" << s.iparams[0] << " row_elems=" << s.iparams[1] << " updates=" << s.iparams[2]; break;
      case Step::JOIN: os << "join"; break;
      case Step::ALL_GATHER: os << "all_gather " << s.bytes << " bytes per partition, rows=" << s.iparams[0]; break;
      case Step::ALL_REDUCE:
        os << (s.overlapped ? "overlapped " : "") << "all_reduce " << s.bytes << " bytes in@" << prog.slots[s.args[0]].offset << " out@" << prog.slots[s.args[1]].offset;
        break;
      default: os << "step";
    }
    os << " args=[";
    for (size_t k = 0; k < s.args.size() && k < 16; k++) os << (k ? "," : "") << s.args[k];
    os << "]\n";
    for (auto& sp : s.sub) dump_plan(prog, *sp, os, indent + 2);
  }
}

uint64_t fnv1a(const std::string& s) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
  return h;
}

}  // namespace

std::unique_ptr<CompiledProgram> compile_module(Module& m, const CompileOptions& opts) {
  auto prog = std::make_unique<CompiledProgram>();
  prog->name = m.name.empty() ? "main" : m.name;
  if (m.attrs.count("mhlo.num_partitions")) prog->num_partitions = (int)attr_int(m.attrs.at("mhlo.num_partitions"));
  if (m.attrs.count("mhlo.num_replicas")) prog->num_replicas = (int)attr_int(m.attrs.at("mhlo.num_replicas"));
  Func* f = m.main();
  Inliner inl(m);
  inl.run(f->body.get());
  fix_region_operands(f->body.get(), inl);
  SkinnyWeightHoist(m).run(f->body.get());
  DecodeAttentionFusion(m).run(f->body.get());
  // unsupported-op check names every offender at once (src/pjrt_plugin/stablehlo_parser.cc:167-184)
  std::set<std::string> bad;
  collect_unsupported(f->body.get(), bad, false);
  if (!bad.empty()) {
    std::string msg = "Unsupported operations for the B200 plugin (no CPU fallback exists):";
    for (auto& b : bad) msg += " " + b;
    throw CompileError(msg);
  }
  Planner pl(*prog, opts, m);
  pl.partition_id = opts.partition_id;
  prog->arena_bytes.push_back(0);
  Block* body = f->body.get();
  for (size_t k = 0; k < body->args.size(); k++) {
    Value* a = body->args[k];
    prog->arg_types.push_back(a->type);
    TensorType t = a->type;
    if (t.dt == DT::TOKEN) { t.dt = DT::U8; t.dims.clear(); }
    int s = pl.new_slot(Slot::ARG, t, 0);
    prog->slots[s].index = (int)k;
    pl.slot_of[a] = s;
  }
  Op* ret = body->ops.empty() ? nullptr : body->ops.back().get();
  if (!ret || ret->name != "func.return") throw CompileError("entry function does not end in func.return");
  std::vector<Value*> rets;
  for (auto* v : ret->operands) rets.push_back(inl.res(v));
  pl.plan_block(body, prog->main, 0, rets);
  pl.hoist_all_reduce_buckets(prog->main);
  // results: a TEMP defined by main becomes the result buffer itself; anything else is copied
  std::set<int> claimed;
  for (size_t k = 0; k < rets.size(); k++) {
    ResultInfo ri;
    ri.type = rets[k]->type;
    if (ri.type.dt == DT::TOKEN) { ri.type.dt = DT::U8; ri.type.dims.clear(); }
    int s = pl.slot_of.at(rets[k]);
    if (prog->slots[s].kind == Slot::TEMP && prog->slots[s].arena == 0 && !claimed.count(s)) {
      prog->slots[s].kind = Slot::RESULT;
      prog->slots[s].index = (int)k;
      claimed.insert(s);
      ri.slot = s;
    } else {
      int rs = pl.new_slot(Slot::RESULT, ri.type, 0);
      prog->slots[rs].index = (int)k;
      Step c;
      c.kind = Step::MEMCPY;
      c.label = "result copy";
      c.args = {rs, s};
      c.bytes = ri.type.bytes();
      prog->main.steps.push_back(std::move(c));
      ri.slot = rs;
    }
    // donation hints (jax: tf.aliasing_output = k / jax.buffer_donor = true)
    for (size_t a = 0; a < f->arg_attrs.size(); a++) {
      auto it = f->arg_attrs[a].find("tf.aliasing_output");
      if (it != f->arg_attrs[a].end() && attr_int(it->second) == (int64_t)k) ri.donated_arg = (int)a;
    }
    prog->results.push_back(ri);
  }
  pl.layout_arena(prog->main);
  // kernels that ended up inside bundles only are not compiled on their own
  {
    std::set<int> used;
    std::function<void(const Plan&)> mark = [&](const Plan& p) {
      for (auto& s : p.steps) {
        if (s.kind == Step::KERNEL) used.insert(s.kernel);
        for (auto& sp : s.sub) mark(*sp);
      }
    };
    mark(prog->main);
    for (size_t k = 0; k < prog->kernels.size(); k++)
      if (!used.count((int)k)) prog->kernels[k].body = "extern \"C\" __global__ void " + prog->kernels[k].name + "() {}\n";
  }
  // static launch count
  {
    bool dynamic = false;
    std::function<long long(const Plan&)> count = [&](const Plan& p) -> long long {
      long long n = 0;
      for (auto& s : p.steps) {
        if (s.kind == Step::KERNEL || s.kind == Step::ALL_REDUCE || s.kind == Step::ALL_GATHER) n += 1;
        else if (s.kind == Step::SCATTER) n += (s.iparams.size() > 5 && s.iparams[5] == 1) ? scatter_elems_launches(s.iparams[0]) - (s.iparams[4] < 0 ? 1 : 0) : scatter_rows_launches(s.iparams[0], s.iparams[2]);
        else if (s.kind == Step::IGEMM) n += s.ig.split_k > 1 ? 2 : 1;
        else if (s.kind == Step::GEMM16) n += (s.g16.path == 0 && s.g16.split_k > 1) ? 2 : 1;
        else if (s.kind == Step::REPACK16) n += (s.iparams[0] + 65534) / 65535;
        else if (s.kind == Step::TRANSPOSE) n += 1;
        else if (s.kind == Step::WHILE) {
          if (s.trip_count < 0) { dynamic = true; continue; }
          n += s.trip_count * count(*s.sub[1]);      // a counted loop never evaluates its condition
        } else if (s.kind == Step::CASE) dynamic = true;
      }
      return n;
    };
    long long n = count(prog->main);
    prog->launches_per_execute = dynamic ? -1 : (int)n;
  }
  std::ostringstream os;
  os << "program " << prog->name << ": " << prog->kernels.size() << " generated kernels, " << prog->slots.size()
     << " slots, arena0 " << prog->arena_bytes[0] << " bytes\n";
  dump_plan(*prog, prog->main, os, 2);
  prog->dump = os.str();
  std::string all;
  for (auto& k : prog->kernels) all += k.body;
  char buf[32];
  snprintf(buf, sizeof buf, "%016llx", (unsigned long long)fnv1a(all + prog->dump));
  prog->fingerprint = buf;
  return prog;
}

}  // namespace b200
