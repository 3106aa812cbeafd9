// The MLIR C API surface of include/mlir_c_b200.h: the builder subset MIGraphX drives rocMLIR with
// (mlir/test/CAPI/mixr_full.c:30-347), a reader for the textual form of the same graphs, the three MIGraphX pipelines
// (mlir/include/mlir-c/Dialect/MIGraphX.h:60-78) and the getters (mlir/lib/CAPI/Dialect/MIGraphX.cpp:54-132), backed
// by a small operation graph and by this library's kernels instead of MLIR and a compiler.
//
// The high-level pipeline is a matcher, not a lowering: it finds the one contraction of the kernel function
// (migraphx.dot / quant_dot / convolution / quant_convolution), reads layouts off the strides of the
// !migraphx.shaped argument types (the role of MIGraphXToTosa's boundary handling, MIGraphXToTosa.cpp:241-275), and
// folds the elementwise ops between the contraction and the return into an RbEpilogue in the fixed step order that
// struct documents; anything it cannot place makes the pipeline fail, which callers treat as "not applicable".
// Host-only code.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "../../include/mlir_c_b200.h"
#include "../../include/rocmlir_b200_tuning.h"
#include "lib_state.h"
#include "problem.h"

namespace rb {
namespace mlirc {

// ---- types and attributes: immutable, interned for the life of the process (as MLIR uniques them in a context) -----
struct Type {
  enum Kind { F32, F16, BF16, F8E4M3, F8E5M2, I1, I8, I32, I64, Index, Shaped, Tensor, Function, Other } kind = Other;
  std::vector<int64_t> shape, strides;   // Shaped / Tensor
  const Type* elem = nullptr;
  std::vector<const Type*> inputs, results;   // Function
  std::string text;                      // canonical spelling
};
struct Attr {
  enum Kind { Unit, Int, Float, String, Array, TypeAttr, DenseSplat, Raw } kind = Raw;
  int64_t i = 0;
  double f = 0;
  std::string s;
  std::vector<const Attr*> elems;
  const Type* type = nullptr;
};

std::mutex g_intern_mu;
std::map<std::string, std::unique_ptr<Type>> g_types;
std::vector<std::unique_ptr<Attr>> g_attrs;
std::set<std::string> g_idents;

const Type* intern(Type t) {
  std::lock_guard<std::mutex> lock(g_intern_mu);
  auto it = g_types.find(t.text);
  if (it != g_types.end()) return it->second.get();
  auto p = std::make_unique<Type>(std::move(t));
  const Type* r = p.get();
  g_types[r->text] = std::move(p);
  return r;
}
const Attr* keep(Attr a) {
  std::lock_guard<std::mutex> lock(g_intern_mu);
  g_attrs.push_back(std::make_unique<Attr>(std::move(a)));
  return g_attrs.back().get();
}
const Type* scalar(Type::Kind k) {
  static const char* names[] = {"f32", "f16", "bf16", "f8E4M3FN", "f8E5M2", "i1", "i8", "i32", "i64", "index"};
  Type t;
  t.kind = k;
  t.text = names[(int)k];
  return intern(t);
}
std::string dims_text(const std::vector<int64_t>& v) {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) s += (i ? "x" : "") + std::to_string(v[i]);
  return s;
}
const Type* shaped(const std::vector<int64_t>& shape, const std::vector<int64_t>& strides, const Type* elem) {
  Type t;
  t.kind = Type::Shaped;
  t.shape = shape; t.strides = strides; t.elem = elem;
  t.text = "!migraphx.shaped<" + dims_text(shape) + (shape.empty() ? "" : "x") + elem->text + ", " + dims_text(strides) + ">";
  return intern(t);
}
const Type* tensor(const std::vector<int64_t>& shape, const Type* elem) {
  Type t;
  t.kind = Type::Tensor;
  t.shape = shape; t.elem = elem;
  t.text = "tensor<" + dims_text(shape) + (shape.empty() ? "" : "x") + elem->text + ">";
  return intern(t);
}

// ---- the operation graph ------------------------------------------------------------------------------------------
struct Operation;
struct Block;
struct Value {
  const Type* type = nullptr;
  Operation* def = nullptr;   // defining op, or null for a block argument
  Block* block = nullptr;     // owning block of a block argument
  int index = 0;
};
struct Region { std::vector<Block*> blocks; Operation* parent = nullptr; ~Region(); };
struct Block { std::vector<Value*> args; std::vector<Operation*> ops; Region* parent = nullptr; ~Block(); };

// What the high-level pipeline made of a kernel function.
struct EpiRecipe {
  uint32_t flags = 0;
  float alpha = 0, out_recip = 0, clip_lo = 0, clip_hi = 0, in_zero = 0;
  int out_zero = 0, mid_type = 0, bias_type = 0, res_type = 0, unary = 0;
  int bias_arg = -1, scale_arg = -1, res_arg = -1;   // function-argument indices of the device vectors
};
struct Lowered {
  int kind = 0;                 // kGemmKind / kConvKind
  RbGemmProblem gemm{};
  RbConvProblem conv{};
  EpiRecipe epi;
  int out_type = -1;            // element type of the result after the epilogue
  int arg_a = -1, arg_b = -1;   // function arguments feeding the contraction (gemm: a, b; conv: input, filter)
  // an operand that arrives as packed int4 (migraphx.unpack, optionally followed by dequantizelinear with a literal
  // scale / zero point): one pass writes it in the contraction's element type into the workspace first
  struct Int4Operand {
    bool on = false;
    int is_unsigned = 0, out_type = -1, zero = 0;
    float scale = 1.0f;
    long long packed_bytes = 0;
    size_t out_bytes = 0;
  } int4_a, int4_b;
  int nargs = 0;                // function arguments (the result follows them in the kernel's argument list)
  std::vector<const Type*> arg_types;   // arguments then results
  std::string name, arch, perf_config;
  uint32_t variant = 0;
  bool applicable = false, compiled = false;
  uint32_t block = 0, grid = 0;
};
enum { kGemmKind = 1, kConvKind = 2 };

struct Operation {
  std::string name;
  std::vector<Value*> operands;
  std::vector<Value*> results;
  std::vector<std::pair<std::string, const Attr*>> attrs;
  std::vector<Region*> regions;
  Block* parent = nullptr;
  std::unique_ptr<Lowered> lowered;   // on the module operation
  std::string diagnostic;             // on the module operation
  ~Operation() {
    for (Value* v : results) delete v;
    for (Region* r : regions) delete r;
  }
  const Attr* attr(const std::string& key) const {
    for (auto& kv : attrs)
      if (kv.first == key) return kv.second;
    return nullptr;
  }
  void set_attr(const std::string& key, const Attr* a) {
    for (auto& kv : attrs)
      if (kv.first == key) { kv.second = a; return; }
    attrs.emplace_back(key, a);
  }
};
Region::~Region() { for (Block* b : blocks) delete b; }
Block::~Block() {
  for (Operation* o : ops) delete o;
  for (Value* v : args) delete v;
}

struct PassManager {
  std::vector<int> stages;   // 1 high level, 2 applicability, 3 backend
  std::string arch;
};

// ---- a small recursive-descent reader shared by mlirAttributeParseGet, mlirTypeParseGet and mlirModuleCreateParse -----
struct Reader {
  const char* p;
  const char* end;
  std::string error;
  explicit Reader(const char* s, size_t n) : p(s), end(s + n) {}
  void ws() {
    while (p < end) {
      if (isspace((unsigned char)*p)) ++p;
      else if (p + 1 < end && p[0] == '/' && p[1] == '/') { while (p < end && *p != '\n') ++p; }
      else break;
    }
  }
  bool at_end() { ws(); return p >= end; }
  bool peek(char c) { ws(); return p < end && *p == c; }
  bool eat(char c) { ws(); if (p < end && *p == c) { ++p; return true; } return false; }
  bool eat(const char* s) {
    ws();
    const size_t n = strlen(s);
    if ((size_t)(end - p) >= n && strncmp(p, s, n) == 0) { p += n; return true; }
    return false;
  }
  bool fail(const std::string& m) { if (error.empty()) error = m + " near '" + std::string(p, std::min<size_t>(24, end - p)) + "'"; return false; }
  static bool ident_char(char c) { return isalnum((unsigned char)c) || c == '_' || c == '.' || c == '$' || c == '-'; }
  std::string ident() {
    ws();
    const char* b = p;
    while (p < end && ident_char(*p)) ++p;
    return std::string(b, p);
  }
  bool integer(int64_t* out) {
    ws();
    const char* b = p;
    if (p < end && (*p == '-' || *p == '+')) ++p;
    const char* d = p;
    while (p < end && isdigit((unsigned char)*p)) ++p;
    if (p == d) { p = b; return false; }
    *out = strtoll(std::string(b, p).c_str(), nullptr, 10);
    return true;
  }
  // number: integer or float; is_float tells which
  bool number(double* f, int64_t* i, bool* is_float) {
    ws();
    const char* b = p;
    if (p < end && (*p == '-' || *p == '+')) ++p;
    const char* d = p;
    while (p < end && isdigit((unsigned char)*p)) ++p;
    bool fl = false;
    if (p < end && *p == '.' ) { fl = true; ++p; while (p < end && isdigit((unsigned char)*p)) ++p; }
    if (p == d) { p = b; return false; }
    if (p < end && (*p == 'e' || *p == 'E')) {
      const char* save = p;
      ++p;
      if (p < end && (*p == '-' || *p == '+')) ++p;
      if (p < end && isdigit((unsigned char)*p)) { fl = true; while (p < end && isdigit((unsigned char)*p)) ++p; }
      else p = save;
    }
    const std::string t(b, p);
    *is_float = fl;
    *f = strtod(t.c_str(), nullptr);
    *i = fl ? (int64_t)*f : strtoll(t.c_str(), nullptr, 10);
    return true;
  }

  const Type* scalar_type(const std::string& id) {
    if (id == "f32") return scalar(Type::F32);
    if (id == "f16") return scalar(Type::F16);
    if (id == "bf16") return scalar(Type::BF16);
    if (id == "f8E4M3FN") return scalar(Type::F8E4M3);
    if (id == "f8E5M2") return scalar(Type::F8E5M2);
    if (id == "i1") return scalar(Type::I1);
    if (id == "i8" || id == "si8") return scalar(Type::I8);
    if (id == "i32" || id == "si32") return scalar(Type::I32);
    if (id == "i64" || id == "si64") return scalar(Type::I64);
    if (id == "index") return scalar(Type::Index);
    return nullptr;
  }
  // "1x64x56x56xf32" -> dims + element type (dimension list may be empty: "f32")
  bool dims_and_elem(std::vector<int64_t>* dims, const Type** elem) {
    for (;;) {
      ws();
      const char* save = p;
      int64_t v;
      if (integer(&v) && p < end && *p == 'x') { ++p; dims->push_back(v); continue; }
      p = save;
      break;
    }
    const std::string id = ident();
    *elem = scalar_type(id);
    return *elem ? true : fail("unknown element type '" + id + "'");
  }
  bool dim_list(std::vector<int64_t>* dims) {   // "200704x3136x56x1" or "0"
    for (;;) {
      int64_t v;
      if (!integer(&v)) return fail("expected a stride list");
      dims->push_back(v);
      if (p < end && *p == 'x') { ++p; continue; }
      return true;
    }
  }
  // `short_shaped`: inside a migraphx op's type list the dialect prefix is dropped ("<1x5x4xf32, 20x4x1>")
  const Type* type(bool short_shaped = false) {
    ws();
    if (eat("!migraphx.shaped") || (short_shaped && peek('<'))) {
      if (!eat('<')) { fail("expected '<'"); return nullptr; }
      std::vector<int64_t> shape, strides;
      const Type* elem = nullptr;
      if (!dims_and_elem(&shape, &elem)) return nullptr;
      if (!eat(',')) { fail("expected ',' before the strides"); return nullptr; }
      if (!shape.empty() && !dim_list(&strides)) return nullptr;
      if (shape.empty()) { int64_t z; integer(&z); }
      if (!eat('>')) { fail("expected '>'"); return nullptr; }
      if (strides.size() != shape.size()) { fail("shape and strides differ in rank"); return nullptr; }
      return shaped(shape, strides, elem);
    }
    if (eat("tensor")) {
      if (!eat('<')) { fail("expected '<'"); return nullptr; }
      std::vector<int64_t> shape;
      const Type* elem = nullptr;
      if (!dims_and_elem(&shape, &elem)) return nullptr;
      if (!eat('>')) { fail("expected '>'"); return nullptr; }
      return tensor(shape, elem);
    }
    if (peek('(')) {   // function type
      Type t;
      t.kind = Type::Function;
      if (!type_list_paren(&t.inputs)) return nullptr;
      if (!eat("->")) { fail("expected '->'"); return nullptr; }
      if (peek('(')) { if (!type_list_paren(&t.results)) return nullptr; }
      else { const Type* r = type(); if (!r) return nullptr; t.results.push_back(r); }
      t.text = "(";
      for (size_t i = 0; i < t.inputs.size(); ++i) t.text += (i ? ", " : "") + t.inputs[i]->text;
      t.text += ") -> (";
      for (size_t i = 0; i < t.results.size(); ++i) t.text += (i ? ", " : "") + t.results[i]->text;
      t.text += ")";
      return intern(t);
    }
    const char* save = p;
    const std::string id = ident();
    if (const Type* s = scalar_type(id)) return s;
    p = save;
    if (p < end && *p == '!') {   // an opaque dialect type (!mhal.token ...): keep its spelling
      const char* b = p;
      ++p;
      while (p < end && (ident_char(*p))) ++p;
      if (p < end && *p == '<') { int depth = 0; do { if (*p == '<') ++depth; if (*p == '>') --depth; ++p; } while (p < end && depth > 0); }
      Type t;
      t.kind = Type::Other;
      t.text = std::string(b, p);
      return intern(t);
    }
    fail("expected a type");
    return nullptr;
  }
  bool type_list_paren(std::vector<const Type*>* out) {
    if (!eat('(')) return fail("expected '('");
    if (eat(')')) return true;
    for (;;) {
      const Type* t = type();
      if (!t) return false;
      out->push_back(t);
      attr_dict_skip();   // argument attributes inside a function type's spelling
      if (eat(',')) continue;
      return eat(')') ? true : fail("expected ')'");
    }
  }
  void attr_dict_skip() {
    ws();
    if (p < end && *p == '{') { std::vector<std::pair<std::string, const Attr*>> tmp; attr_dict(&tmp); }
  }

  const Attr* attribute() {
    ws();
    Attr a;
    if (eat('[')) {
      a.kind = Attr::Array;
      if (!eat(']')) {
        for (;;) {
          const Attr* e = attribute();
          if (!e) return nullptr;
          a.elems.push_back(e);
          if (eat(',')) continue;
          if (!eat(']')) { fail("expected ']'"); return nullptr; }
          break;
        }
      }
      return keep(a);
    }
    if (peek('"')) {
      ++p;
      const char* b = p;
      while (p < end && *p != '"') ++p;
      a.kind = Attr::String;
      a.s = std::string(b, p);
      if (p < end) ++p;
      return keep(a);
    }
    if (eat("dense")) {
      if (!eat('<')) { fail("expected '<' after dense"); return nullptr; }
      bool is_float;
      if (eat("true")) { a.i = 1; a.f = 1; is_float = false; }
      else if (eat("false")) { a.i = 0; a.f = 0; is_float = false; }
      else {
        // a one-element list, dense<[0.25]>, is the same splat (mlir/test/fusion/pr-e2e/mixr-dot-int4-f16.mlir:9)
        const bool bracket = eat('[');
        if (!number(&a.f, &a.i, &is_float)) { fail("only splat dense attributes are read"); return nullptr; }
        if (bracket && !eat(']')) { fail("only splat (one-value) dense attributes are read"); return nullptr; }
      }
      if (!eat('>')) { fail("only splat dense attributes are read"); return nullptr; }
      if (!eat(':')) { fail("expected ':' after dense<>"); return nullptr; }
      a.kind = Attr::DenseSplat;
      a.type = type();
      return a.type ? keep(a) : nullptr;
    }
    if (eat("unit")) { a.kind = Attr::Unit; return keep(a); }
    if (eat("true")) { a.kind = Attr::Int; a.i = 1; a.type = scalar(Type::I1); return keep(a); }
    if (eat("false")) { a.kind = Attr::Int; a.i = 0; a.type = scalar(Type::I1); return keep(a); }
    {
      bool is_float;
      const char* save = p;
      if (number(&a.f, &a.i, &is_float)) {
        a.kind = is_float ? Attr::Float : Attr::Int;
        ws();
        if (p < end && *p == ':' ) { ++p; a.type = type(); if (!a.type) return nullptr; }
        return keep(a);
      }
      p = save;
    }
    if (peek('(') || peek('!') || (p < end && isalpha((unsigned char)*p))) {
      const char* save = p;
      const Type* t = type();
      if (t) { a.kind = Attr::TypeAttr; a.type = t; return keep(a); }
      p = save;
      error.clear();
    }
    if (p < end && (*p == '@' || *p == '#')) {   // symbol references and dialect attributes are kept as text
      const char* b = p;
      ++p;
      while (p < end && (ident_char(*p) || *p == ':')) ++p;
      if (p < end && *p == '<') { int depth = 0; do { if (*p == '<') ++depth; if (*p == '>') --depth; ++p; } while (p < end && depth > 0); }
      a.kind = Attr::Raw;
      a.s = std::string(b, p);
      return keep(a);
    }
    fail("expected an attribute");
    return nullptr;
  }
  bool attr_dict(std::vector<std::pair<std::string, const Attr*>>* out) {
    if (!eat('{')) return fail("expected '{'");
    if (eat('}')) return true;
    for (;;) {
      ws();
      std::string key;
      if (peek('"')) { ++p; const char* b = p; while (p < end && *p != '"') ++p; key = std::string(b, p); if (p < end) ++p; }
      else key = ident();
      if (key.empty()) return fail("expected an attribute name");
      const Attr* v;
      if (eat('=')) { v = attribute(); if (!v) return false; }
      else { Attr u; u.kind = Attr::Unit; v = keep(u); }
      out->emplace_back(key, v);
      if (eat(',')) continue;
      return eat('}') ? true : fail("expected '}'");
    }
  }
};

// ---- module text ------------------------------------------------------------------------------------------------------
struct ModuleParser {
  Reader r;
  std::map<std::string, Value*> values;
  explicit ModuleParser(const char* s, size_t n) : r(s, n) {}

  Operation* parse_module() {
    auto mod = std::make_unique<Operation>();
    mod->name = "builtin.module";
    Region* reg = new Region;
    reg->parent = mod.get();
    Block* body = new Block;
    body->parent = reg;
    reg->blocks.push_back(body);
    mod->regions.push_back(reg);
    bool braced = false;
    if (r.eat("module")) {
      r.ws();
      if (r.peek('@')) { ++r.p; r.ident(); }
      if (r.eat("attributes")) { if (!r.attr_dict(&mod->attrs)) return nullptr; }
      if (!r.eat('{')) { r.fail("expected '{' after module"); return nullptr; }
      braced = true;
    }
    if (!parse_body(body, braced)) return nullptr;
    return mod.release();
  }
  // ops of a module body: functions and nested modules
  bool parse_body(Block* body, bool braced) {
    for (;;) {
      if (r.at_end()) return braced ? r.fail("missing '}'") : true;
      if (braced && r.eat('}')) return true;
      if (r.eat("func.func")) {
        Operation* f = parse_func();
        if (!f) return false;
        f->parent = body;
        body->ops.push_back(f);
        continue;
      }
      if (r.eat("module")) {   // a nested module (the kernel copy under @__xmodule_): its functions join the search
        auto nested = std::make_unique<Operation>();
        nested->name = "builtin.module";
        r.ws();
        if (r.peek('@')) { ++r.p; r.ident(); }
        if (r.eat("attributes")) { if (!r.attr_dict(&nested->attrs)) return false; }
        if (!r.eat('{')) return r.fail("expected '{' after module");
        Region* reg = new Region;
        reg->parent = nested.get();
        Block* nb = new Block;
        nb->parent = reg;
        reg->blocks.push_back(nb);
        nested->regions.push_back(reg);
        if (!parse_body(nb, true)) return false;
        nested->parent = body;
        body->ops.push_back(nested.release());
        continue;
      }
      return r.fail("expected func.func or module");
    }
  }
  Operation* parse_func() {
    auto f = std::make_unique<Operation>();
    f->name = "func.func";
    if (r.eat("private")) { Attr a; a.kind = Attr::String; a.s = "private"; f->set_attr("sym_visibility", keep(a)); }
    else if (r.eat("public")) {}
    if (!r.eat('@')) { r.fail("expected '@' and a function name"); return nullptr; }
    Attr nm; nm.kind = Attr::String; nm.s = r.ident();
    f->set_attr("sym_name", keep(nm));
    if (!r.eat('(')) { r.fail("expected '('"); return nullptr; }
    Region* reg = new Region;
    reg->parent = f.get();
    Block* body = new Block;
    body->parent = reg;
    reg->blocks.push_back(body);
    f->regions.push_back(reg);
    values.clear();
    Type ft;
    ft.kind = Type::Function;
    if (!r.eat(')')) {
      for (;;) {
        if (!r.eat('%')) { r.fail("expected an argument name"); return nullptr; }
        const std::string an = r.ident();
        if (!r.eat(':')) { r.fail("expected ':'"); return nullptr; }
        const Type* t = r.type();
        if (!t) return nullptr;
        r.attr_dict_skip();
        Value* v = new Value;
        v->type = t; v->block = body; v->index = (int)body->args.size();
        body->args.push_back(v);
        values[an] = v;
        ft.inputs.push_back(t);
        if (r.eat(',')) continue;
        if (!r.eat(')')) { r.fail("expected ')'"); return nullptr; }
        break;
      }
    }
    if (r.eat("->")) {
      if (r.peek('(')) {
        if (!r.eat('(')) return nullptr;
        for (;;) {
          const Type* t = r.type();
          if (!t) return nullptr;
          r.attr_dict_skip();
          ft.results.push_back(t);
          if (r.eat(',')) continue;
          if (!r.eat(')')) { r.fail("expected ')'"); return nullptr; }
          break;
        }
      } else {
        const Type* t = r.type();
        if (!t) return nullptr;
        ft.results.push_back(t);
      }
    }
    ft.text = "fn" + std::to_string((uintptr_t)f.get());
    Attr fta; fta.kind = Attr::TypeAttr; fta.type = intern(ft);
    f->set_attr("function_type", keep(fta));
    if (r.eat("attributes")) { if (!r.attr_dict(&f->attrs)) return nullptr; }
    if (!r.peek('{')) return f.release();   // a declaration
    r.eat('{');
    for (;;) {
      if (r.eat('}')) break;
      if (r.at_end()) { r.fail("missing '}' of the function"); return nullptr; }
      Operation* op = parse_op();
      if (!op) return nullptr;
      op->parent = body;
      body->ops.push_back(op);
    }
    return f.release();
  }
  Value* lookup(const std::string& n) {
    auto it = values.find(n);
    return it == values.end() ? nullptr : it->second;
  }
  // One operation in the custom assembly the migraphx dialect prints:
  //   %r = migraphx.op %a, %b {attrs} : <types> -> <type>      migraphx.literal (dense<..> : tensor<..>) : <type>
  //   return %r : type                                          %t, %r = mhal.launch @f (%a, ...) : (types) -> type
  Operation* parse_op() {
    auto op = std::make_unique<Operation>();
    std::vector<std::string> result_names;
    while (r.peek('%')) {
      ++r.p;
      result_names.push_back(r.ident());
      if (r.eat(',')) continue;
      if (!r.eat('=')) { r.fail("expected '='"); return nullptr; }
      break;
    }
    op->name = r.ident();
    if (op->name == "return") op->name = "func.return";
    if (op->name.empty()) { r.fail("expected an operation name"); return nullptr; }
    const bool mixr = op->name.rfind("migraphx.", 0) == 0;
    if (r.peek('@')) { ++r.p; Attr a; a.kind = Attr::Raw; a.s = "@" + r.ident(); op->set_attr("callee", keep(a)); }
    if (r.peek('(') && mixr) {   // migraphx.literal (value)
      r.eat('(');
      const Attr* v = r.attribute();
      if (!v) return nullptr;
      if (!r.eat(')')) { r.fail("expected ')'"); return nullptr; }
      op->set_attr("value", v);
    } else {
      const bool paren = r.eat('(');
      while (r.peek('%')) {
        ++r.p;
        const std::string n = r.ident();
        Value* v = lookup(n);
        if (!v) { r.fail("use of undefined value %" + n); return nullptr; }
        op->operands.push_back(v);
        if (!r.eat(',')) break;
      }
      if (paren && !r.eat(')')) { r.fail("expected ')'"); return nullptr; }
    }
    if (r.peek('{')) { if (!r.attr_dict(&op->attrs)) return nullptr; }
    std::vector<const Type*> result_types;
    if (r.eat(':')) {
      if (op->name == "func.return" || !mixr) {
        // generic tail: operand types, optionally "-> result types"; only the results matter here
        std::vector<const Type*> tys;
        if (r.peek('(')) { if (!r.type_list_paren(&tys)) return nullptr; }
        else { do { const Type* t = r.type(); if (!t) return nullptr; tys.push_back(t); } while (r.eat(',')); }
        if (r.eat("->")) {
          if (r.peek('(')) { if (!r.type_list_paren(&result_types)) return nullptr; }
          else { do { const Type* t = r.type(); if (!t) return nullptr; result_types.push_back(t); } while (r.eat(',')); }
        }
      } else {
        std::vector<const Type*> tys;
        do { const Type* t = r.type(true); if (!t) return nullptr; tys.push_back(t); } while (r.eat(','));
        if (r.eat("->")) {
          do { const Type* t = r.type(true); if (!t) return nullptr; result_types.push_back(t); } while (r.eat(','));
        } else {
          result_types = tys;   // "migraphx.literal (...) : <type>": the one type is the result's
        }
      }
    }
    for (size_t i = 0; i < result_names.size(); ++i) {
      Value* v = new Value;
      // ops with more results than listed types (mhal.launch's token) get an opaque type for the extras
      const size_t extra = result_names.size() - std::min(result_names.size(), result_types.size());
      v->type = i < extra ? nullptr : result_types[i - extra];
      v->def = op.get();
      v->index = (int)i;
      op->results.push_back(v);
      values[result_names[i]] = v;
    }
    return op.release();
  }
};

// ---- cloning ------------------------------------------------------------------------------------------------------------
Operation* clone_op(const Operation* o, std::map<const Value*, Value*>& remap);
Block* clone_block(const Block* b, std::map<const Value*, Value*>& remap) {
  Block* n = new Block;
  for (const Value* a : b->args) {
    Value* v = new Value(*a);
    v->block = n;
    n->args.push_back(v);
    remap[a] = v;
  }
  for (const Operation* o : b->ops) {
    Operation* c = clone_op(o, remap);
    c->parent = n;
    n->ops.push_back(c);
  }
  return n;
}
Operation* clone_op(const Operation* o, std::map<const Value*, Value*>& remap) {
  Operation* n = new Operation;
  n->name = o->name;
  n->attrs = o->attrs;
  n->diagnostic = o->diagnostic;
  if (o->lowered) n->lowered = std::make_unique<Lowered>(*o->lowered);
  for (const Value* v : o->operands) {
    auto it = remap.find(v);
    n->operands.push_back(it == remap.end() ? const_cast<Value*>(v) : it->second);
  }
  for (const Value* v : o->results) {
    Value* c = new Value(*v);
    c->def = n;
    n->results.push_back(c);
    remap[v] = c;
  }
  for (const Region* r : o->regions) {
    Region* nr = new Region;
    nr->parent = n;
    for (const Block* b : r->blocks) {
      Block* nb = clone_block(b, remap);
      nb->parent = nr;
      nr->blocks.push_back(nb);
    }
    n->regions.push_back(nr);
  }
  return n;
}

// ---- printing (mlirOperationDump) -----------------------------------------------------------------------------------------
std::string attr_text(const Attr* a) {
  switch (a->kind) {
    case Attr::Unit: return "unit";
    case Attr::Int: return std::to_string(a->i) + (a->type ? " : " + a->type->text : "");
    case Attr::Float: { char b[64]; snprintf(b, sizeof(b), "%g", a->f); return std::string(b) + (a->type ? " : " + a->type->text : ""); }
    case Attr::String: return "\"" + a->s + "\"";
    case Attr::Array: { std::string s = "["; for (size_t i = 0; i < a->elems.size(); ++i) s += (i ? ", " : "") + attr_text(a->elems[i]); return s + "]"; }
    case Attr::TypeAttr: return a->type->text;
    case Attr::DenseSplat: { char b[64]; snprintf(b, sizeof(b), "%g", a->f); return "dense<" + std::string(b) + "> : " + a->type->text; }
    default: return a->s;
  }
}
void dump_op(const Operation* o, int indent, std::map<const Value*, std::string>& names, std::string* out) {
  const std::string pad(indent, ' ');
  *out += pad;
  for (size_t i = 0; i < o->results.size(); ++i) {
    const std::string n = "%" + std::to_string(names.size());
    names[o->results[i]] = n;
    *out += (i ? ", " : "") + n;
  }
  if (!o->results.empty()) *out += " = ";
  *out += "\"" + o->name + "\"(";
  for (size_t i = 0; i < o->operands.size(); ++i) *out += (i ? ", " : "") + (names.count(o->operands[i]) ? names[o->operands[i]] : std::string("%?"));
  *out += ")";
  if (!o->attrs.empty()) {
    *out += " {";
    for (size_t i = 0; i < o->attrs.size(); ++i) *out += (i ? ", " : "") + o->attrs[i].first + " = " + attr_text(o->attrs[i].second);
    *out += "}";
  }
  for (const Region* r : o->regions) {
    *out += " ({\n";
    for (const Block* b : r->blocks) {
      if (!b->args.empty()) {
        *out += pad + "^bb(";
        for (size_t i = 0; i < b->args.size(); ++i) {
          const std::string n = "%arg" + std::to_string(i);
          names[b->args[i]] = n;
          *out += (i ? ", " : "") + n + ": " + (b->args[i]->type ? b->args[i]->type->text : "?");
        }
        *out += "):\n";
      }
      for (const Operation* c : b->ops) dump_op(c, indent + 2, names, out);
    }
    *out += pad + "})";
  }
  *out += " : (";
  for (size_t i = 0; i < o->operands.size(); ++i) *out += (i ? ", " : "") + (o->operands[i]->type ? o->operands[i]->type->text : std::string("?"));
  *out += ") -> (";
  for (size_t i = 0; i < o->results.size(); ++i) *out += (i ? ", " : "") + (o->results[i]->type ? o->results[i]->type->text : std::string("?"));
  *out += ")\n";
}

// ---- the high-level pipeline: graph -> problem + epilogue ---------------------------------------------------------------------
int rb_type_of(const Type* t) {
  switch (t->kind) {
    case Type::F32: return RB_F32;
    case Type::F16: return RB_F16;
    case Type::BF16: return RB_BF16;
    case Type::I8: return RB_I8;
    case Type::I32: return RB_I32;
    case Type::F8E4M3: return RB_F8E4M3;
    case Type::F8E5M2: return RB_F8E5M2;
    default: return -1;
  }
}
void find_kernel_funcs(Operation* module, std::vector<Operation*>* out) {
  for (Region* r : module->regions)
    for (Block* b : r->blocks)
      for (Operation* o : b->ops) {
        if (o->name == "func.func" && !o->regions.empty() && !o->regions[0]->blocks.empty() && !o->regions[0]->blocks[0]->ops.empty())
          out->push_back(o);
        else if (o->name == "builtin.module") find_kernel_funcs(o, out);
      }
}
// The function a module is about: the one carrying `kernel` (in a nested kernel module first), else the only one.
Operation* kernel_func(Operation* module) {
  std::vector<Operation*> fs;
  find_kernel_funcs(module, &fs);
  Operation* pick = nullptr;
  for (Operation* f : fs)
    if (f->attr("kernel")) pick = f;   // the last one: nested kernel modules come after the host wrappers
  if (!pick && fs.size() == 1) pick = fs[0];
  return pick;
}

// How a value of the elementwise tail relates to the function's arguments.
struct Source {
  enum Kind { None, Arg, Literal, Chain } kind = None;
  int arg = -1;
  double lit = 0;
  const Type* type = nullptr;      // the value's own type (after broadcasts)
  const Type* base = nullptr;      // the argument's / literal's type before broadcasting
  // an argument seen through migraphx.unpack (int4 pairs -> i8) and perhaps dequantizelinear: still kind Arg
  bool unpacked = false, dequantized = false;
  int is_unsigned = 0, zero = 0;
  float scale = 1.0f;
};

struct Matcher {
  Operation* func;
  Block* body;
  Lowered* L;
  std::string err;
  std::map<const Value*, Source> src;
  int stage = 0;   // position in the epilogue's fixed step order reached so far

  bool fail(const std::string& m) { if (err.empty()) err = m; return false; }
  bool step(int s, const char* what) {
    if (s <= stage) return fail(std::string(what) + " comes after a later step of the fused epilogue's fixed order");
    stage = s;
    return true;
  }
  static bool ints(const Attr* a, std::vector<int64_t>* out) {
    if (!a || a->kind != Attr::Array) return false;
    for (const Attr* e : a->elems) { if (e->kind != Attr::Int) return false; out->push_back(e->i); }
    return true;
  }
  // dims of a shaped type sorted by stride, largest first (memory order); stable for equal strides
  static std::vector<int> memory_order(const Type* t) {
    std::vector<int> idx(t->shape.size());
    for (size_t i = 0; i < idx.size(); ++i) idx[i] = (int)i;
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return t->strides[a] > t->strides[b]; });
    return idx;
  }
  static bool dense_in(const Type* t, const std::vector<int>& order) {
    int64_t acc = 1;
    for (int i = (int)order.size() - 1; i >= 0; --i) {
      const int d = order[i];
      if (t->shape[d] != 1 && t->strides[d] != acc) return false;
      acc *= t->shape[d];
    }
    return true;
  }

  // [batch...] x R x C matrix stored row-major (trans = 0) or column-major (trans = 1), batches dense outside
  bool matrix(const Type* t, int* g, int* rows, int* cols, int* trans, bool* batch_shared = nullptr) {
    if (!t || t->kind != Type::Shaped || t->shape.size() < 2) return fail("a dot operand must be a shaped tensor of rank >= 2");
    const size_t n = t->shape.size();
    int64_t G = 1;
    for (size_t i = 0; i + 2 < n; ++i) G *= t->shape[i];
    const int64_t R = t->shape[n - 2], C = t->shape[n - 1];
    const int64_t sr = t->strides[n - 2], sc = t->strides[n - 1];
    if ((sc == 1 || C == 1) && (sr == C || R == 1)) *trans = 0;
    else if ((sr == 1 || R == 1) && (sc == R || C == 1)) *trans = 1;
    else return fail("a dot operand must be a dense row-major or column-major matrix (strides " + dims_text(t->strides) + ")");
    // one matrix shared by every batch (a multibroadcast along the batch dimensions: stride 0)
    bool shared = G > 1;
    for (size_t i = 0; i + 2 < n; ++i)
      if (t->shape[i] != 1 && t->strides[i] != 0) shared = false;
    if (batch_shared) *batch_shared = shared;
    int64_t acc = R * C;
    for (int i = (int)n - 3; i >= 0 && !shared; --i) {
      if (t->shape[i] != 1 && t->strides[i] != acc) return fail("batch dimensions of a dot operand must be dense (or broadcast with stride 0)");
      acc *= t->shape[i];
    }
    if (shared && !batch_shared) return fail("only the second dot operand may be shared between the batches");
    if (G > 0x7fffffff || R > 0x7fffffff || C > 0x7fffffff) return fail("extent exceeds 2^31");
    *g = (int)G; *rows = (int)R; *cols = (int)C;
    return true;
  }

  // logical (n, c, h, w)-style tensor -> layout string over `letters` (logical order) with the group letter inserted
  // before the channel letter `ch`
  // A 1-D convolution (rank-3 tensors n, c, w) is the 2-D one with a unit image height, as MIGraphX itself expands it
  // (mlir/lib/Conversion/MIGraphXToTosa/MIGraphXToTosa.cpp:241-275): the unit dimension goes in front of the width.
  static Type with_unit_height(const Type* t) {
    Type u = *t;
    if (u.shape.size() == 3) {
      u.shape.insert(u.shape.begin() + 2, 1);
      u.strides.insert(u.strides.begin() + 2, t->strides[2] * t->shape[2]);
    }
    return u;
  }

  bool conv_layout(const Type* t0, const char* letters, char ch, int64_t groups, char* out8) {
    if (!t0 || t0->kind != Type::Shaped || (t0->shape.size() != 4 && t0->shape.size() != 3))
      return fail("convolution tensors must be shaped tensors of rank 4 (or 3: one image dimension)");
    const Type expanded = with_unit_height(t0);
    const Type* t = &expanded;
    const std::vector<int> order = memory_order(t);
    if (!dense_in(t, order)) return fail("convolution tensors must be dense in some dimension order (strides " + dims_text(t->strides) + ")");
    if (groups > 1 && t->shape[strchr(letters, ch) - letters] % groups) return fail("channels are not divisible by the group count");
    std::string s;
    for (int d : order) {
      if (letters[d] == ch) s += 'g';
      s += letters[d];
    }
    snprintf(out8, 8, "%s", s.c_str());
    return true;
  }

  // which dimensions of a broadcast operand vary: returns per-dimension "varies" flags for a value of `like`'s rank
  static std::vector<bool> varying(const Type* t) {
    std::vector<bool> v(t->shape.size());
    for (size_t i = 0; i < v.size(); ++i) v[i] = t->strides[i] != 0 && t->shape[i] != 1;
    return v;
  }

  bool run() {
    // 1. classify every value
    for (Value* a : body->args) { Source s; s.kind = Source::Arg; s.arg = a->index; s.type = a->type; s.base = a->type; src[a] = s; }
    Operation* contraction = nullptr;
    Value* chain = nullptr;
    Value* returned = nullptr;
    const Type* acc_type = nullptr;   // element type of the value flowing down the chain
    for (Operation* o : body->ops) {
      const std::string& n = o->name;
      if (n == "func.return") {
        if (o->operands.size() != 1) return fail("the kernel function must return one value");
        returned = o->operands[0];
        continue;
      }
      if (n == "migraphx.literal") {
        const Attr* v = o->attr("value");
        if (!v || v->kind != Attr::DenseSplat) return fail("only splat literals are supported");
        Source s; s.kind = Source::Literal; s.lit = v->f; s.type = o->results[0]->type; s.base = v->type;
        src[o->results[0]] = s;
        continue;
      }
      if (n == "migraphx.multibroadcast" || n == "migraphx.broadcast") {
        Source s = src[o->operands[0]];
        if (s.kind != Source::Arg && s.kind != Source::Literal) return fail(n + " of a computed value is not fused");
        s.type = o->results[0]->type;
        src[o->results[0]] = s;
        continue;
      }
      if (n == "migraphx.unpack") {
        // MIGraphX.td:183-212: doubles `axis` by splitting every byte into its two 4-bit values
        Source s = src[o->operands[0]];
        const Type* it = o->operands[0]->type;
        const Type* ot = o->results[0]->type;
        const Attr* ax = o->attr("axis");
        const Attr* un = o->attr("isUnsigned");
        if (s.kind != Source::Arg || s.unpacked || s.type != s.base) return fail("unpack must read a function argument directly");
        if (!ax || ax->kind != Attr::Int || !it || it->kind != Type::Shaped || ax->i != (int64_t)it->shape.size() - 1 ||
            it->strides.back() != 1 || !ot || ot->shape.back() != 2 * it->shape.back())
          return fail("unpack is supported along the last, contiguous dimension");
        const std::vector<int> order = memory_order(it);
        if (!dense_in(it, order)) return fail("the packed tensor must be dense");
        s.unpacked = true;
        s.is_unsigned = un && ((un->kind == Attr::Int && un->i != 0) || (un->kind == Attr::Raw && un->s == "true") ||
                               (un->kind == Attr::String && un->s == "true")) ? 1 : 0;
        s.type = ot;
        src[o->results[0]] = s;
        continue;
      }
      if (n == "migraphx.dequantizelinear" && !chain && !o->operands.empty() && src[o->operands[0]].kind == Source::Arg &&
          src[o->operands[0]].unpacked) {
        Source s = src[o->operands[0]];
        if (s.dequantized) return fail("an operand is dequantised once");
        double sc = 1.0, zp = 0.0;
        if (o->operands.size() < 2 || !literal_of(o->operands[1], &sc)) return fail("the scale of an int4 operand must be a literal");
        if (o->operands.size() > 2 && !literal_of(o->operands[2], &zp)) return fail("the zero point of an int4 operand must be a literal");
        s.dequantized = true;
        s.scale = (float)sc;
        s.zero = (int)zp;
        s.type = o->results[0]->type;
        src[o->results[0]] = s;
        continue;
      }
      const bool is_contraction = n == "migraphx.dot" || n == "migraphx.quant_dot" || n == "migraphx.convolution" ||
                                  n == "migraphx.quant_convolution";
      if (is_contraction) {
        if (contraction) return fail("more than one contraction in the kernel function");
        if (o->operands.size() != 2 || src[o->operands[0]].kind != Source::Arg || src[o->operands[1]].kind != Source::Arg)
          return fail("the operands of " + n + " must be function arguments");
        contraction = o;
        if (!lower_contraction(o)) return false;
        chain = o->results[0];
        Source s; s.kind = Source::Chain; s.type = chain->type;
        src[chain] = s;
        acc_type = chain->type->elem;
        continue;
      }
      // an op of the elementwise tail: one operand is the chain value
      if (!chain) return fail("operation " + n + " before the contraction (input fusion is not supported)");
      int ci = -1;
      for (size_t i = 0; i < o->operands.size(); ++i)
        if (o->operands[i] == chain) ci = (int)i;
      if (ci < 0) return fail("operation " + n + " does not continue the contraction's result");
      if (o->results.size() != 1 || !o->results[0]->type || o->results[0]->type->kind != Type::Shaped)
        return fail("operation " + n + " must produce one shaped tensor");
      if (!fold(o, ci, &acc_type)) return false;
      chain = o->results[0];
      Source s; s.kind = Source::Chain; s.type = chain->type;
      src[chain] = s;
    }
    if (!contraction) return fail("no contraction (dot / quant_dot / convolution / quant_convolution) in the kernel function");
    if (returned != chain) return fail("the function must return the fused chain's last value");
    // result type and storage
    const Type* rt = chain->type;
    L->out_type = rb_type_of(rt->elem);
    if (L->out_type < 0) return fail("unsupported result element type " + rt->elem->text);
    if (L->kind == kGemmKind) {
      int g, m, n2, tc;
      if (!matrix(rt, &g, &m, &n2, &tc)) return false;
      const bool folded = (long long)g * m == (long long)L->gemm.g * L->gemm.m && g != L->gemm.g;   // shared second operand
      if (folded && tc) return fail("a second operand shared between the batches needs a row-major result");
      if (folded && (L->epi.flags & RB_EPI_BIAS_ROW)) return fail("a per-row bias cannot follow a dot whose batch is folded into its rows");
      if ((!folded && (g != L->gemm.g || m != L->gemm.m)) || n2 != L->gemm.n) return fail("the result's shape does not match the dot");
      L->gemm.trans_c = tc;
      L->gemm.c_type = L->out_type;
    } else {
      if (!conv_layout(rt, "nkhw", 'k', L->conv.g, L->conv.out_layout)) return false;
    }
    // the contraction's declared type rounds the accumulator before float steps (f16 dot -> add runs in f16)
    const int mid = rb_type_of(contraction->results[0]->type->elem);
    if (L->epi.flags && (mid == RB_F16 || mid == RB_BF16)) { L->epi.flags |= RB_EPI_ROUND_MID; L->epi.mid_type = mid; }
    if (L->kind == kGemmKind && L->gemm.ab_type == RB_I8 && L->epi.flags == 0 && L->out_type != RB_I32)
      return fail("quant_dot without a dequantisation must return i32");
    // kernel arguments: the function's arguments, then its result
    for (Value* a : body->args) L->arg_types.push_back(a->type);
    L->arg_types.push_back(rt);
    L->nargs = (int)body->args.size();
    // every argument must have been used by something the kernel reads
    std::set<int> used = {L->arg_a, L->arg_b};
    if (L->epi.bias_arg >= 0) used.insert(L->epi.bias_arg);
    if (L->epi.scale_arg >= 0) used.insert(L->epi.scale_arg);
    if (L->epi.res_arg >= 0) used.insert(L->epi.res_arg);
    if ((int)used.size() != L->nargs) return fail("a function argument is not consumed by the fused kernel");
    return true;
  }

  bool lower_contraction(Operation* o) {
    const Value* x = o->operands[0];
    const Value* y = o->operands[1];
    const int tx = rb_type_of(x->type->elem), ty = rb_type_of(y->type->elem);
    const int tr = rb_type_of(o->results[0]->type->elem);
    if (tx < 0 || ty < 0 || tr < 0) return fail("unsupported element type in " + o->name);
    const bool quant = o->name == "migraphx.quant_dot" || o->name == "migraphx.quant_convolution";
    if (quant ? !(tx == RB_I8 && ty == RB_I8 && tr == RB_I32) : false) return fail(o->name + " takes i8 operands and produces i32");
    if (o->name == "migraphx.dot" || o->name == "migraphx.quant_dot") {
      L->kind = kGemmKind;
      RbGemmProblem& p = L->gemm;
      int g1, m, k, ta, g2, k2, n, tb;
      bool b_shared = false;
      if (!matrix(x->type, &g1, &m, &k, &ta) || !matrix(y->type, &g2, &k2, &n, &tb, &b_shared)) return false;
      if (g1 != g2 || k != k2) return fail("dot operands do not agree in batch or reduction extent");
      p.g = g1; p.m = m; p.n = n; p.k = k;
      if (b_shared) {
        // G x M x K times one K x N matrix is the (G * M) x K x N product on the same bytes when A is stored row by row
        // (broadcast batch operands: mlir/lib/Conversion/MIGraphXToTosa/MIGraphXToTosa.cpp:393-440)
        if (ta) return fail("a second operand shared between the batches needs a row-major first operand");
        if ((long long)g1 * m > 0x7fffffffLL) return fail("extent exceeds 2^31");
        p.g = 1; p.m = g1 * m;
      }
      p.trans_a = ta;          // A stored G x K x M when column-major
      p.trans_b = tb;          // B logical K x N: column-major storage is the library's trans_b (G x N x K)
      if (tx == ty) p.ab_type = tx;
      else if (tx == RB_F8E4M3 && ty == RB_F8E5M2) p.ab_type = RB_F8E4M3_E5M2;
      else if (tx == RB_F8E5M2 && ty == RB_F8E4M3) p.ab_type = RB_F8E5M2_E4M3;
      else return fail("dot operands of different element types");
      p.c_type = tr;
      L->arg_a = src[x].arg; L->arg_b = src[y].arg;
      for (int side = 0; side < 2; ++side) {
        const Source& s = src[side ? y : x];
        Lowered::Int4Operand& q = side ? L->int4_b : L->int4_a;
        q.on = s.unpacked;
        if (!s.unpacked) continue;
        const Type* ot = (side ? y : x)->type;
        q.is_unsigned = s.is_unsigned; q.zero = s.zero; q.scale = s.scale;
        q.out_type = rb_type_of(ot->elem);
        if (!s.dequantized && q.out_type != RB_I8) return fail("an unpacked int4 operand without dequantizelinear is i8");
        long long elems = 1;
        for (int64_t d : ot->shape) elems *= d;
        q.packed_bytes = elems / 2;
        q.out_bytes = (size_t)elems * dtype_bytes(q.out_type);
      }
      return true;
    }
    if (src[x].unpacked || src[y].unpacked) return fail("int4 operands are supported for dot, not for convolutions");
    L->kind = kConvKind;
    RbConvProblem& c = L->conv;
    memset(&c, 0, sizeof(c));
    const size_t rank = x->type->shape.size();
    if ((rank != 4 && rank != 3) || y->type->shape.size() != rank || o->results[0]->type->shape.size() != rank)
      return fail("only 1-D and 2-D convolutions are matched");
    const Type in_t = with_unit_height(x->type), fil_t = with_unit_height(y->type), out_t = with_unit_height(o->results[0]->type);
    const Type* in = &in_t;
    const Type* fil = &fil_t;
    const Type* out = &out_t;
    std::vector<int64_t> pad, stride, dil;
    if (!ints(o->attr("padding"), &pad) || !ints(o->attr("stride"), &stride) || !ints(o->attr("dilation"), &dil))
      return fail("convolution needs padding, stride and dilation attributes");
    if (rank == 3) {   // one image dimension: [pad_l, pad_r] (or [pad]), [stride], [dilation]
      if (pad.size() == 1) pad = {pad[0], pad[0]};
      if (pad.size() != 2 || stride.size() != 1 || dil.size() != 1) return fail("1-D convolution attributes of the wrong length");
      pad = {0, pad[0], 0, pad[1]};
      stride = {1, stride[0]};
      dil = {1, dil[0]};
    }
    if (pad.size() == 2) pad = {pad[0], pad[1], pad[0], pad[1]};
    if (pad.size() != 4 || stride.size() != 2 || dil.size() != 2) return fail("convolution attributes of the wrong length");
    const Attr* ga = o->attr("group");
    const int64_t groups = ga && ga->kind == Attr::Int ? ga->i : 1;
    if (groups <= 0 || in->shape[1] % groups || fil->shape[0] % groups) return fail("bad group count");
    if (fil->shape[1] * groups != in->shape[1]) return fail("filter channels do not match the input's");
    c.n = (int)in->shape[0]; c.g = (int)groups; c.c = (int)(in->shape[1] / groups); c.k = (int)(fil->shape[0] / groups);
    c.h = (int)in->shape[2]; c.w = (int)in->shape[3]; c.y = (int)fil->shape[2]; c.x = (int)fil->shape[3];
    c.stride_h = (int)stride[0]; c.stride_w = (int)stride[1]; c.dil_h = (int)dil[0]; c.dil_w = (int)dil[1];
    c.pad_h = (int)pad[0]; c.pad_w = (int)pad[1]; c.pad_h_r = (int)pad[2]; c.pad_w_r = (int)pad[3];
    c.ho = (int)out->shape[2]; c.wo = (int)out->shape[3];
    if (out->shape[0] != in->shape[0] || out->shape[1] != fil->shape[0]) return fail("the convolution's result shape is inconsistent");
    c.data_type = tx;
    c.direction = 0;
    if (tx != ty) return fail("convolution operands of different element types");
    if (!conv_layout(in, "nchw", 'c', groups, c.in_layout) || !conv_layout(fil, "kcyx", 'k', groups, c.fil_layout)) return false;
    // the raw result's layout: the final value's layout is taken in run(); start from the contraction's own
    if (!conv_layout(out, "nkhw", 'k', groups, c.out_layout)) return false;
    L->arg_a = src[x].arg; L->arg_b = src[y].arg;
    return true;
  }

  // the channel / column dimension of the chain value
  int col_dim(const Type* t) const { return L->kind == kGemmKind ? (int)t->shape.size() - 1 : 1; }
  int row_dim(const Type* t) const { return L->kind == kGemmKind ? (int)t->shape.size() - 2 : -1; }

  bool literal_of(const Value* v, double* out) {
    const Source& s = src[v];
    if (s.kind != Source::Literal) return false;
    *out = s.lit;
    return true;
  }

  bool fold(Operation* o, int ci, const Type** acc_type) {
    const std::string& n = o->name;
    EpiRecipe& e = L->epi;
    const Type* rt = o->results[0]->type;
    if (n == "migraphx.relu") { if (!step(60, "relu")) return false; e.flags |= RB_EPI_RELU; *acc_type = rt->elem; return true; }
    {
      // the other unary elementwise ops (MIGraphX.td:134-181): one of them, where the rectifier would stand
      static const char* const kUnary[] = {"", "abs", "ceil", "erf", "exp", "floor", "log", "neg", "recip", "rsqrt", "sigmoid", "sqrt", "tanh"};
      for (int u = 1; u <= RB_UNARY_TANH; ++u) {
        if (n != std::string("migraphx.") + kUnary[u]) continue;
        if (o->operands.size() != 1) return fail(n + " takes one operand");
        if (rb_type_of(rt->elem) == RB_I8 || rb_type_of(rt->elem) == RB_I32) return fail(n + " is fused on floating-point values only");
        if (!step(55, kUnary[u])) return false;
        e.flags |= RB_EPI_UNARY;
        e.unary = u;
        *acc_type = rt->elem;
        return true;
      }
    }
    if (n == "migraphx.clip") {
      double lo, hi;
      if (ci != 0 || o->operands.size() != 3 || !literal_of(o->operands[1], &lo) || !literal_of(o->operands[2], &hi))
        return fail("clip bounds must be literals");
      if (!step(70, "clip")) return false;
      e.flags |= RB_EPI_CLIP; e.clip_lo = (float)lo; e.clip_hi = (float)hi;
      return true;
    }
    if (n == "migraphx.convert") { if (!step(95, "convert")) return false; *acc_type = rt->elem; return true; }   // the store converts
    if (n == "migraphx.add" || n == "migraphx.mul") {
      if (o->operands.size() != 2) return fail(n + " takes two operands");
      const Value* other = o->operands[1 - ci];
      const Source& s = src[other];
      if (n == "migraphx.mul") {
        if (s.kind != Source::Literal) return fail("mul is fused only with a literal (a per-tensor scale)");
        if (!step(30, "mul")) return false;
        e.flags |= RB_EPI_ALPHA; e.alpha = (float)s.lit;
        return true;
      }
      if (s.kind != Source::Arg) return fail("add is fused only with a function argument (bias vector or same-shape tensor)");
      const Type* bt = s.type;
      if (!bt || bt->kind != Type::Shaped || bt->shape.size() != rt->shape.size()) return fail("add operands differ in rank");
      for (size_t i = 0; i < bt->shape.size(); ++i)   // extents of 1 broadcast implicitly
        if (bt->shape[i] != rt->shape[i] && bt->shape[i] != 1) return fail("add operands differ in shape");
      const std::vector<bool> var = varying(bt);
      int nvar = 0;
      for (bool b : var) nvar += b;
      const int elem = rb_type_of(bt->elem);
      if (!(elem == RB_F32 || elem == RB_F16 || elem == RB_BF16)) return fail("add operand must be f32, f16 or bf16");
      bool full = bt->shape == rt->shape;
      for (size_t i = 0; i < var.size(); ++i) full = full && (var[i] || bt->shape[i] == 1);
      if (full && bt->strides == o->operands[ci]->type->strides && s.base == bt) {   // same-shape, same-layout operand
        if (!step(50, "same-shape add")) return false;
        e.flags |= RB_EPI_RESIDUAL; e.res_arg = s.arg; e.res_type = elem;
        return true;
      }
      if (!step(40, "broadcast add")) return false;
      e.flags |= RB_EPI_BIAS; e.bias_arg = s.arg; e.bias_type = elem;
      if (nvar == 0) { e.flags |= RB_EPI_BIAS_SCALAR; return true; }
      if (nvar == 1 && var[col_dim(bt)]) return true;
      if (nvar == 1 && row_dim(bt) >= 0 && var[row_dim(bt)]) { e.flags |= RB_EPI_BIAS_ROW; return true; }
      return fail("the broadcast of the add operand is not per channel / per column, per row or scalar");
    }
    if (n == "migraphx.dequantizelinear") {
      if (ci != 0 || o->operands.size() < 2) return fail("dequantizelinear must take the contraction's result as its input");
      if (o->operands.size() == 3) {
        double zp;
        if (!literal_of(o->operands[2], &zp)) return fail("the dequantisation zero point must be a literal");
        if (zp != 0) { if (!step(10, "dequantizelinear zero point")) return false; e.flags |= RB_EPI_ZP_IN; e.in_zero = (float)zp; }
      }
      const Source& s = src[o->operands[1]];
      if (s.kind == Source::Literal) {
        if (!step(30, "dequantizelinear")) return false;
        e.flags |= RB_EPI_ALPHA; e.alpha = (float)s.lit;
      } else if (s.kind == Source::Arg) {
        const std::vector<bool> var = varying(s.type);
        int nvar = 0;
        for (bool b : var) nvar += b;
        if (!(nvar == 1 && var[col_dim(s.type)]) || rb_type_of(s.type->elem) != RB_F32)
          return fail("a dequantisation scale tensor must be f32 and per channel / per column");
        if (!step(35, "dequantizelinear")) return false;
        e.flags |= RB_EPI_COL_SCALE; e.scale_arg = s.arg;
      } else return fail("the dequantisation scale must be a literal or a function argument");
      *acc_type = rt->elem;
      return true;
    }
    if (n == "migraphx.quantizelinear") {
      double scale, zp = 0;
      if (ci != 0 || o->operands.size() < 2 || !literal_of(o->operands[1], &scale)) return fail("the quantisation scale must be a literal");
      if (o->operands.size() == 3 && !literal_of(o->operands[2], &zp)) return fail("the quantisation zero point must be a literal");
      if (rb_type_of(rt->elem) != RB_I8) return fail("quantizelinear must produce i8");
      if (!step(80, "quantizelinear")) return false;
      e.flags |= RB_EPI_REQUANT;
      e.out_recip = 1.0f / (float)scale;   // tosa.reciprocal then tosa.mul in f32 (MIGraphXToTosa.cpp:917-921)
      if (zp != 0) { e.flags |= RB_EPI_ZP_OUT; e.out_zero = (int)zp; }
      *acc_type = rt->elem;
      return true;
    }
    return fail("operation " + n + " is not part of the fused elementwise tail");
  }
};

Operation* module_of(MlirModule m) { return const_cast<Operation*>(static_cast<const Operation*>(m.ptr)); }

bool run_high_level(Operation* mod) {
  Operation* f = kernel_func(mod);
  if (!f) { mod->diagnostic = "no kernel function in the module"; return false; }
  auto L = std::make_unique<Lowered>();
  Matcher mt{f, f->regions[0]->blocks[0], L.get()};
  if (!mt.run()) { mod->diagnostic = mt.err; return false; }
  const Attr* nm = f->attr("sym_name");
  L->name = nm && nm->kind == Attr::String ? nm->s : "main";
  for (const char* key : {"arch", "mhal.arch"}) {
    const Attr* a = f->attr(key);
    if (!a) a = mod->attr(key);
    if (a && a->kind == Attr::String && L->arch.empty()) L->arch = a->s;
  }
  const Attr* pc = f->attr("perf_config");
  if (pc && pc->kind == Attr::String) L->perf_config = pc->s;
  if (mod->lowered) { L->perf_config = mod->lowered->perf_config; L->variant = mod->lowered->variant; }   // tuning set earlier
  mod->lowered = std::move(L);
  mod->diagnostic.clear();
  return true;
}

// the GEMM the module's kernel runs as (a convolution's implicit GEMM included)
bool gemm_of(const Lowered& L, RbGemmProblem* gp) {
  if (L.kind == kGemmKind) { *gp = L.gemm; return true; }
  return rbConvGetGemmProblem(&L.conv, gp) == RB_SUCCESS;
}

bool run_applicability(Operation* mod) {
  if (!mod->lowered) { mod->diagnostic = "run the high-level pipeline first"; return false; }
  Lowered& L = *mod->lowered;
  L.applicable = false;
  if (!L.perf_config.empty() && !perf_config_to_variant(L.perf_config.c_str(), &L.variant)) {
    mod->diagnostic = "perf_config '" + L.perf_config + "' does not name a tile configuration of this library";
    return false;
  }
  RbGemmProblem gp;
  const int saved = rbGetGemmVariant();
  rbSetGemmVariant((int)L.variant);
  RbGemmConfigInfo info;
  const bool ok = gemm_of(L, &gp) && rbGemmGetConfig(&gp, &info) == RB_SUCCESS;
  rbSetGemmVariant(saved);
  if (!ok) { mod->diagnostic = std::string("no kernel for the problem: ") + rbGetLastError(); return false; }
  if (L.variant) {   // an explicit configuration must be one the problem can really take
    const uint32_t want_ctas = L.variant & 0xF, want_bn = (L.variant >> 12) & 0xF;
    const uint32_t bn_code = info.tile_n == 64 ? 1u : info.tile_n == 128 ? 2u : 3u;
    if ((want_ctas && want_ctas != (uint32_t)info.ctas) || (want_bn && want_bn != bn_code)) {
      mod->diagnostic = "the tile configuration of perf_config '" + L.perf_config + "' is not applicable to this problem";
      return false;
    }
  }
  L.block = info.block;
  L.grid = info.grid;
  L.applicable = true;
  mod->diagnostic.clear();
  return true;
}

bool arch_ok(const std::string& a) {
  return a == "sm_100a" || a == "sm_100" || a == "nvptx64-nvidia-cuda:sm_100a" || a == "nvptx64-nvidia-cuda:sm_100";
}

bool run_backend(Operation* mod, const std::string& arch) {
  if (!arch_ok(arch)) { mod->diagnostic = "architecture '" + arch + "' is not sm_100a"; return false; }
  if (!mod->lowered && !run_high_level(mod)) return false;
  if (!run_applicability(mod)) return false;
  mod->lowered->compiled = true;
  return true;
}

RbStatus build_epilogue(const Lowered& L, void* const* args, RbEpilogue* e, bool* have) {
  memset(e, 0, sizeof(*e));
  const EpiRecipe& r = L.epi;
  e->flags = r.flags; e->alpha = r.alpha; e->out_recip = r.out_recip; e->mid_type = r.mid_type; e->bias_type = r.bias_type;
  e->clip_lo = r.clip_lo; e->clip_hi = r.clip_hi; e->in_zero = r.in_zero; e->out_zero = r.out_zero; e->res_type = r.res_type; e->unary = r.unary;
  if (r.bias_arg >= 0) e->bias = args[r.bias_arg];
  if (r.scale_arg >= 0) e->col_scale = static_cast<const float*>(args[r.scale_arg]);
  if (r.res_arg >= 0) e->residual = args[r.res_arg];
  *have = r.flags != 0;
  return RB_SUCCESS;
}

}  // namespace mlirc
}  // namespace rb

using namespace rb;
using namespace rb::mlirc;

// ---- C entry points ------------------------------------------------------------------------------------------------------------
extern "C" {

MlirStringRef mlirStringRefCreateFromCString(const char* str) { return mlirStringRefCreate(str, str ? strlen(str) : 0); }

MlirContext mlirContextCreate(void) { return MlirContext{new int(1)}; }
void mlirContextDestroy(MlirContext c) { delete static_cast<int*>(c.ptr); }
MlirLocation mlirLocationUnknownGet(MlirContext c) { return MlirLocation{c.ptr}; }

MlirType mlirF32TypeGet(MlirContext) { return MlirType{scalar(Type::F32)}; }
MlirType mlirF16TypeGet(MlirContext) { return MlirType{scalar(Type::F16)}; }
MlirType mlirBF16TypeGet(MlirContext) { return MlirType{scalar(Type::BF16)}; }
MlirType mlirFloat8E4M3FNTypeGet(MlirContext) { return MlirType{scalar(Type::F8E4M3)}; }
MlirType mlirFloat8E5M2TypeGet(MlirContext) { return MlirType{scalar(Type::F8E5M2)}; }
MlirType mlirIntegerTypeGet(MlirContext, unsigned bits) {
  return MlirType{bits == 1 ? scalar(Type::I1) : bits == 8 ? scalar(Type::I8) : bits == 32 ? scalar(Type::I32) : bits == 64 ? scalar(Type::I64) : nullptr};
}
MlirType mlirTypeParseGet(MlirContext, MlirStringRef s) {
  Reader r(s.data, s.length);
  const Type* t = r.type();
  return MlirType{t && r.at_end() ? t : nullptr};
}
MlirType rocmlirMIXRShapedTypeGet(intptr_t rank, const int64_t* shape, const int64_t* strides, MlirType elem) {
  if (!elem.ptr || rank < 0) return MlirType{nullptr};
  return MlirType{shaped(std::vector<int64_t>(shape, shape + rank), std::vector<int64_t>(strides, strides + rank),
                         static_cast<const Type*>(elem.ptr))};
}
bool rocmlirIsAMIXRShapedType(MlirType t) { return t.ptr && static_cast<const Type*>(t.ptr)->kind == Type::Shaped; }
MlirType rocmlirMIXRShapedTypeAsTensor(MlirType t) {
  const Type* s = static_cast<const Type*>(t.ptr);
  return MlirType{s && s->kind == Type::Shaped ? tensor(s->shape, s->elem) : nullptr};
}

MlirAttribute mlirAttributeParseGet(MlirContext, MlirStringRef s) {
  Reader r(s.data, s.length);
  const Attr* a = r.attribute();
  return MlirAttribute{a && r.at_end() ? a : nullptr};
}
MlirAttribute mlirUnitAttrGet(MlirContext) { Attr a; a.kind = Attr::Unit; return MlirAttribute{keep(a)}; }
MlirAttribute mlirStringAttrGet(MlirContext, MlirStringRef s) { Attr a; a.kind = Attr::String; a.s = std::string(s.data, s.length); return MlirAttribute{keep(a)}; }
MlirAttribute mlirIntegerAttrGet(MlirType t, int64_t v) { Attr a; a.kind = Attr::Int; a.i = v; a.type = static_cast<const Type*>(t.ptr); return MlirAttribute{keep(a)}; }
MlirIdentifier mlirIdentifierGet(MlirContext, MlirStringRef s) {
  std::lock_guard<std::mutex> lock(g_intern_mu);
  return MlirIdentifier{&*g_idents.insert(std::string(s.data, s.length)).first};
}
MlirNamedAttribute mlirNamedAttributeGet(MlirIdentifier name, MlirAttribute attr) { return MlirNamedAttribute{name, attr}; }

MlirModule mlirModuleCreateEmpty(MlirLocation) {
  Operation* m = new Operation;
  m->name = "builtin.module";
  Region* r = new Region; r->parent = m;
  Block* b = new Block; b->parent = r;
  r->blocks.push_back(b);
  m->regions.push_back(r);
  return MlirModule{m};
}
MlirModule mlirModuleCreateParse(MlirContext, MlirStringRef text) {
  ModuleParser p(text.data, text.length);
  Operation* m = p.parse_module();
  if (!m || !p.r.error.empty()) {
    fail(RB_INVALID_PARAM, "module text: " + p.r.error);   // readable through rbGetLastError
    delete m;
    return MlirModule{nullptr};
  }
  return MlirModule{m};
}
MlirBlock mlirModuleGetBody(MlirModule m) { return MlirBlock{module_of(m)->regions[0]->blocks[0]}; }
MlirOperation mlirModuleGetOperation(MlirModule m) { return MlirOperation{module_of(m)}; }
MlirModule mlirModuleFromOperation(MlirOperation op) {
  Operation* o = static_cast<Operation*>(op.ptr);
  return MlirModule{o && o->name == "builtin.module" ? o : nullptr};
}
void mlirModuleDestroy(MlirModule m) { delete module_of(m); }
MlirRegion mlirRegionCreate(void) { return MlirRegion{new Region}; }
void mlirRegionAppendOwnedBlock(MlirRegion r, MlirBlock b) {
  Region* reg = static_cast<Region*>(r.ptr);
  Block* blk = static_cast<Block*>(b.ptr);
  blk->parent = reg;
  reg->blocks.push_back(blk);
}
MlirBlock mlirBlockCreate(intptr_t n, MlirType const* args, MlirLocation const*) {
  Block* b = new Block;
  for (intptr_t i = 0; i < n; ++i) {
    Value* v = new Value;
    v->type = static_cast<const Type*>(args[i].ptr); v->block = b; v->index = (int)i;
    b->args.push_back(v);
  }
  return MlirBlock{b};
}
MlirValue mlirBlockGetArgument(MlirBlock b, intptr_t pos) {
  Block* blk = static_cast<Block*>(b.ptr);
  return MlirValue{pos >= 0 && pos < (intptr_t)blk->args.size() ? blk->args[pos] : nullptr};
}
void mlirBlockAppendOwnedOperation(MlirBlock b, MlirOperation op) {
  Block* blk = static_cast<Block*>(b.ptr);
  Operation* o = static_cast<Operation*>(op.ptr);
  o->parent = blk;
  blk->ops.push_back(o);
}
void mlirBlockInsertOwnedOperation(MlirBlock b, intptr_t pos, MlirOperation op) {
  Block* blk = static_cast<Block*>(b.ptr);
  Operation* o = static_cast<Operation*>(op.ptr);
  o->parent = blk;
  pos = std::max<intptr_t>(0, std::min<intptr_t>(pos, (intptr_t)blk->ops.size()));
  blk->ops.insert(blk->ops.begin() + pos, o);
}

MlirOperationState mlirOperationStateGet(MlirStringRef name, MlirLocation loc) {
  MlirOperationState s;
  memset(&s, 0, sizeof(s));
  s.name = name;
  s.location = loc;
  return s;
}
#define RB_STATE_APPEND(T, count, array)                                   \
  array = static_cast<T*>(realloc(array, sizeof(T) * (size_t)(count + n)));   \
  memcpy(array + count, items, sizeof(T) * (size_t)n);                      \
  count += n;
void mlirOperationStateAddResults(MlirOperationState* s, intptr_t n, MlirType const* items) { RB_STATE_APPEND(MlirType, s->nResults, s->results) }
void mlirOperationStateAddOperands(MlirOperationState* s, intptr_t n, MlirValue const* items) { RB_STATE_APPEND(MlirValue, s->nOperands, s->operands) }
void mlirOperationStateAddOwnedRegions(MlirOperationState* s, intptr_t n, MlirRegion const* items) { RB_STATE_APPEND(MlirRegion, s->nRegions, s->regions) }
void mlirOperationStateAddAttributes(MlirOperationState* s, intptr_t n, MlirNamedAttribute const* items) { RB_STATE_APPEND(MlirNamedAttribute, s->nAttributes, s->attributes) }
#undef RB_STATE_APPEND

MlirOperation mlirOperationCreate(MlirOperationState* s) {
  Operation* o = new Operation;
  o->name = std::string(s->name.data, s->name.length);
  for (intptr_t i = 0; i < s->nOperands; ++i) o->operands.push_back(const_cast<Value*>(static_cast<const Value*>(s->operands[i].ptr)));
  for (intptr_t i = 0; i < s->nResults; ++i) {
    Value* v = new Value;
    v->type = static_cast<const Type*>(s->results[i].ptr); v->def = o; v->index = (int)i;
    o->results.push_back(v);
  }
  for (intptr_t i = 0; i < s->nAttributes; ++i)
    o->set_attr(*static_cast<const std::string*>(s->attributes[i].name.ptr), static_cast<const Attr*>(s->attributes[i].attribute.ptr));
  for (intptr_t i = 0; i < s->nRegions; ++i) {
    Region* r = static_cast<Region*>(s->regions[i].ptr);
    r->parent = o;
    o->regions.push_back(r);
  }
  free(s->results); free(s->operands); free(s->regions); free(s->attributes); free(s->successors);
  memset(s, 0, sizeof(*s));
  return MlirOperation{o};
}
MlirOperation mlirOperationClone(MlirOperation op) {
  std::map<const Value*, Value*> remap;
  return MlirOperation{clone_op(static_cast<const Operation*>(op.ptr), remap)};
}
void mlirOperationSetAttributeByName(MlirOperation op, MlirStringRef name, MlirAttribute attr) {
  static_cast<Operation*>(op.ptr)->set_attr(std::string(name.data, name.length), static_cast<const Attr*>(attr.ptr));
}
MlirValue mlirOperationGetResult(MlirOperation op, intptr_t pos) {
  Operation* o = static_cast<Operation*>(op.ptr);
  return MlirValue{pos >= 0 && pos < (intptr_t)o->results.size() ? o->results[pos] : nullptr};
}
void mlirOperationDump(MlirOperation op) {
  std::map<const Value*, std::string> names;
  std::string out;
  dump_op(static_cast<const Operation*>(op.ptr), 0, names, &out);
  fputs(out.c_str(), stderr);
}

MlirPassManager mlirPassManagerCreate(MlirContext) { return MlirPassManager{new PassManager}; }
void mlirPassManagerDestroy(MlirPassManager pm) { delete static_cast<PassManager*>(pm.ptr); }
void mlirMIGraphXAddHighLevelPipeline(MlirPassManager pm) { static_cast<PassManager*>(pm.ptr)->stages.push_back(1); }
void mlirMIGraphXAddApplicabilityPipeline(MlirPassManager pm) { static_cast<PassManager*>(pm.ptr)->stages.push_back(2); }
bool mlirMIGraphXAddBackendPipeline(MlirPassManager pm, const char* arch) {
  if (!arch || !arch_ok(arch)) return false;   // MIGraphX.h:66-73: false for an architecture that cannot be targeted
  PassManager* p = static_cast<PassManager*>(pm.ptr);
  p->stages.push_back(3);
  p->arch = arch;
  return true;
}
MlirLogicalResult mlirPassManagerRunOnOp(MlirPassManager pm, MlirOperation op) {
  PassManager* p = static_cast<PassManager*>(pm.ptr);
  Operation* mod = static_cast<Operation*>(op.ptr);
  if (!p || !mod || mod->name != "builtin.module") return MlirLogicalResult{0};
  for (int st : p->stages) {
    const bool ok = st == 1 ? run_high_level(mod) : st == 2 ? run_applicability(mod) : run_backend(mod, p->arch);
    if (!ok) return MlirLogicalResult{0};
  }
  return MlirLogicalResult{1};
}

void mlirGetKernelInfo(MlirModule module, int* size, void* data) {
  Operation* mod = module_of(module);
  if (!size && !data) return;
  std::vector<int> info;
  std::string name = "main";
  if (mod->lowered) {
    name = mod->lowered->name;
    for (const Type* t : mod->lowered->arg_types) {
      info.push_back((int)t->shape.size());
      for (int d : Matcher::memory_order(t)) info.push_back((int)t->shape[d]);
    }
  } else if (Operation* f = kernel_func(mod)) {   // before the high-level pipeline: arguments as declared
    const Attr* nm = f->attr("sym_name");
    if (nm && nm->kind == Attr::String) name = nm->s;
    for (Value* a : f->regions[0]->blocks[0]->args) {
      info.push_back((int)a->type->shape.size());
      for (int d : Matcher::memory_order(a->type)) info.push_back((int)a->type->shape[d]);
    }
  }
  const int nargs = mod->lowered ? (int)mod->lowered->arg_types.size()
                                 : (kernel_func(mod) ? (int)kernel_func(mod)->regions[0]->blocks[0]->args.size() : 0);
  if (!data) {
    *size = (int)((1 + info.size()) * sizeof(int) + name.size());
    return;
  }
  int* out = static_cast<int*>(data);
  out[0] = nargs;
  for (size_t i = 0; i < info.size(); ++i) out[1 + i] = info[i];
  memcpy(out + 1 + info.size(), name.data(), name.size());
}
void mlirGetKernelAttrs(MlirModule module, uint32_t* attrs) {
  Operation* mod = module_of(module);
  if (!attrs || !mod->lowered || !mod->lowered->compiled) return;
  attrs[0] = mod->lowered->block;
  attrs[1] = mod->lowered->grid;
}
bool mlirGetBinary(MlirModule module, size_t* size, char* bin) {
  Operation* mod = module_of(module);
  if ((!size && !bin) || !mod->lowered || !mod->lowered->compiled) return false;
  const void* image = nullptr;
  size_t n = 0;
  if (rbGetKernelBinary(&image, &n) != RB_SUCCESS) return false;
  if (bin) memcpy(bin, image, n);
  else *size = n;
  return true;
}

const char* rbModuleGetDiagnostic(MlirModule module) { return module.ptr ? module_of(module)->diagnostic.c_str() : ""; }

static size_t int4_bytes(const Lowered::Int4Operand& q) { return q.on ? (q.out_bytes + 255) / 256 * 256 : 0; }
static RbStatus module_ready(Operation* mod, size_t nargs) {
  if (!mod || !mod->lowered || !mod->lowered->applicable) return fail(RB_INVALID_PARAM, "run the pipelines on the module first");
  if (nargs != mod->lowered->arg_types.size())
    return fail(RB_INVALID_PARAM, "the kernel takes " + std::to_string(mod->lowered->arg_types.size()) + " pointers (arguments, then the result)");
  return RB_SUCCESS;
}
size_t rbModuleGetWorkspaceSize(MlirModule module) {
  Operation* mod = module_of(module);
  if (!mod || !mod->lowered) return 0;
  const Lowered& L = *mod->lowered;
  const int saved = rbGetGemmVariant();
  rbSetGemmVariant((int)L.variant);
  const size_t n = L.kind == kGemmKind ? rbGemmWorkspaceSize(&L.gemm) : rbConvEpiWorkspaceSize(&L.conv, L.out_type);
  rbSetGemmVariant(saved);
  return n + int4_bytes(L.int4_a) + int4_bytes(L.int4_b);   // unpacked operands first, the kernel's own workspace behind them
}
static RbStatus module_run(MlirModule module, void* const* args, size_t nargs, void* ws, size_t ws_bytes, void* stream, RbKernelLaunch* capture) {
  Operation* mod = module_of(module);
  RbStatus st = module_ready(mod, nargs);
  if (st != RB_SUCCESS) return st;
  const Lowered& L = *mod->lowered;
  for (size_t i = 0; i < nargs; ++i)
    if (!args[i]) return fail(RB_INVALID_PARAM, "argument " + std::to_string(i) + " is NULL");
  RbEpilogue e;
  bool have = false;
  build_epilogue(L, args, &e, &have);
  void* result = args[nargs - 1];
  const void* op_a = args[L.arg_a];
  const void* op_b = args[L.arg_b];
  if (L.int4_a.on || L.int4_b.on) {
    if (capture) return fail(RB_UNSUPPORTED, "a kernel with int4 operands runs an unpacking pass first: it has no single-kernel binary");
    const size_t need = int4_bytes(L.int4_a) + int4_bytes(L.int4_b);
    if (!ws || ws_bytes < need) return fail(RB_WORKSPACE_TOO_SMALL, "workspace of " + std::to_string(rbModuleGetWorkspaceSize(module)) + " bytes required");
    uint8_t* w = static_cast<uint8_t*>(ws);
    for (int side = 0; side < 2; ++side) {
      const Lowered::Int4Operand& q = side ? L.int4_b : L.int4_a;
      if (!q.on) continue;
      st = rbUnpackInt4(side ? op_b : op_a, w, q.packed_bytes, q.is_unsigned, q.out_type, q.scale, q.zero, stream);
      if (st != RB_SUCCESS) return st;
      (side ? op_b : op_a) = w;
      w += int4_bytes(q);
    }
    ws = w;
    ws_bytes -= need;
  }
  const int saved = rbGetGemmVariant();
  rbSetGemmVariant((int)L.variant);
  if (L.kind == kGemmKind) {
    st = capture ? rbGemmEncodeLaunch(&L.gemm, have ? &e : nullptr, op_a, op_b, result, capture)
                 : rbGemm(&L.gemm, have ? &e : nullptr, op_a, op_b, result, ws, ws_bytes, stream);
  } else {
    // kernel-argument order of the library's convolution: (filter, input, output); migraphx.convolution takes (input, filter)
    st = capture ? rbConvEncodeLaunch(&L.conv, have ? &e : nullptr, L.out_type, args[L.arg_b], args[L.arg_a], result, capture)
                 : rbConvEpi(&L.conv, have ? &e : nullptr, L.out_type, args[L.arg_b], args[L.arg_a], result, ws, ws_bytes, stream);
  }
  rbSetGemmVariant(saved);
  return st;
}
RbStatus rbModuleLaunch(MlirModule module, void* const* args, size_t nargs, void* ws, size_t ws_bytes, void* stream) {
  return module_run(module, args, nargs, ws, ws_bytes, stream, nullptr);
}
RbStatus rbModuleGetKernelLaunch(MlirModule module, void* const* args, size_t nargs, RbKernelLaunch* out) {
  if (!out) return fail(RB_INVALID_PARAM, "out is NULL");
  return module_run(module, args, nargs, nullptr, 0, nullptr, out);
}

// ---- tuning: the module's problem behind the library's tuning entry points -----------------------------------------------------
static RbProblem problem_of(Operation* mod) {
  RbProblem none{nullptr};
  if (!mod || !mod->lowered) return none;
  return mod->lowered->kind == kGemmKind ? rbProblemFromGemm(&mod->lowered->gemm) : rbProblemFromConv(&mod->lowered->conv);
}
MlirRockTuningSpace mlirRockTuningSpaceCreate(MlirModule module, RocmlirTuningParamSetKind kind) {
  RbProblem p = problem_of(module_of(module));
  if (!p.ptr) return MlirRockTuningSpace{nullptr};
  RbTuningSpace s = rbTuningSpaceCreate(p, (RbTuningParamSetKind)kind);
  rbProblemDestroy(p);
  return MlirRockTuningSpace{s.ptr};
}
unsigned mlirRockTuningGetNumParams(MlirRockTuningSpace s) { return s.ptr ? rbTuningGetNumParams(RbTuningSpace{s.ptr}) : 0; }
MlirRockTuningParam mlirRockTuningParamCreate(void) { return MlirRockTuningParam{rbTuningParamCreate().ptr}; }
void mlirRockTuningParamDestroy(MlirRockTuningParam p) { rbTuningParamDestroy(RbTuningParam{p.ptr}); }
void mlirRockTuningSpaceDestroy(MlirRockTuningSpace s) { if (s.ptr) rbTuningSpaceDestroy(RbTuningSpace{s.ptr}); }
bool mlirRockTuningParamGet(MlirRockTuningSpace s, unsigned pos, MlirRockTuningParam p) {
  return s.ptr && rbTuningParamGet(RbTuningSpace{s.ptr}, pos, RbTuningParam{p.ptr});
}
bool mlirRockTuningParamGetQuick(MlirRockTuningSpace s, unsigned pos, MlirRockTuningParam p) {
  return s.ptr && rbTuningParamGetQuick(RbTuningSpace{s.ptr}, pos, RbTuningParam{p.ptr});
}
size_t mlirRockTuningParamToString(MlirRockTuningParam p, char* buf, size_t len) { return rbTuningParamToString(RbTuningParam{p.ptr}, buf, len); }
bool mlirRockTuningSetFromStr(MlirModule module, MlirStringRef perf) {
  Operation* mod = module_of(module);
  if (!mod || !mod->lowered) return false;
  const std::string s(perf.data, perf.length);
  uint32_t v = 0;
  if (!perf_config_to_variant(s.c_str(), &v)) return false;
  RbProblem p = problem_of(mod);
  const bool ok = p.ptr && rbTuningSetFromStr(p, s.c_str(), s.size());
  if (p.ptr) rbProblemDestroy(p);
  if (!ok) return false;
  mod->lowered->perf_config = s;
  mod->lowered->variant = v;
  mod->lowered->applicable = mod->lowered->compiled = false;
  return true;
}
bool mlirRockTuningSetParam(MlirModule module, MlirRockTuningParam param) {
  char buf[ROCMLIR_TUNING_PARAM_STRING_BUFSZ];
  const size_t n = rbTuningParamToString(RbTuningParam{param.ptr}, buf, sizeof(buf));
  if (n >= sizeof(buf)) return false;
  return mlirRockTuningSetFromStr(module, mlirStringRefCreate(buf, n));
}
MlirRockTuningTable mlirRockTuningTableCreate(void) { return MlirRockTuningTable{rbTuningTableCreate().ptr}; }
void mlirRockTuningTableDestroy(MlirRockTuningTable t) { rbTuningTableDestroy(RbTuningTable{t.ptr}); }
bool mlirRockTuningUpdateTable(MlirRockTuningTable t, MlirStringRef key, MlirStringRef perf, float time) {
  return rbTuningUpdateTable(RbTuningTable{t.ptr}, key.data, key.length, perf.data, perf.length, time);
}
size_t mlirRockTuningGetKey(MlirModule module, char* buf, size_t len) {
  RbProblem p = problem_of(module_of(module));
  if (!p.ptr) return (size_t)-1;
  const size_t n = rbTuningGetKey(p, buf, len);
  rbProblemDestroy(p);
  return n;
}
bool mlirRockTuningSetFromTable(MlirRockTuningTable t, MlirModule module) {
  Operation* mod = module_of(module);
  RbProblem p = problem_of(mod);
  if (!p.ptr) return false;
  bool ok = rbTuningSetFromTable(RbTuningTable{t.ptr}, p);
  char buf[ROCMLIR_TUNING_PARAM_STRING_BUFSZ] = {0};
  if (ok) {
    const size_t n = rbProblemGetPerfConfig(p, buf, sizeof(buf));
    ok = n < sizeof(buf);
  }
  rbProblemDestroy(p);
  return ok && mlirRockTuningSetFromStr(module, mlirStringRefCreateFromCString(buf));
}
enum RocmlirSplitKSelectionLikelihood mlirIsSplitKFaster(int64_t g, int64_t m, int64_t n, int64_t k, int64_t cus,
                                                         RocmlirTuningParamSetKind level) {
  return (enum RocmlirSplitKSelectionLikelihood)rbIsSplitKFaster(g, m, n, k, cus, (RbTuningParamSetKind)level);
}
bool mlirIsModuleFusible(MlirModule module, MlirStringRef perf) {
  RbProblem p = problem_of(module_of(module));
  if (!p.ptr) return false;
  const bool ok = rbIsProblemFusible(p, perf.data, perf.length);
  rbProblemDestroy(p);
  return ok;
}
size_t mlirGetNumPrefillArgs(MlirModule) { return 0; }   // no kernel of this library accumulates into its output with atomics
void mlirGetPrefillArgsInfo(MlirModule, size_t*, MlirAttribute*, size_t) {}
size_t mlirGetNumAuxBuffers(MlirModule) { return 0; }    // as in the reference (mlir/lib/CAPI/Dialect/Rock.cpp:201-205)
void mlirGetAuxBuffersInfo(MlirModule, size_t*, MlirAttribute*, size_t) {}

}  // extern "C"
