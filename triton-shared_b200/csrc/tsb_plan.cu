// Launch plans on the C side: tsb_plan_create / tsb_launch.
//
// The host side of this package compiles a Triton kernel to a JSON launch plan: a kernel family
// plus parameters that are polynomials over the kernel's scalar arguments, program ids, grid
// sizes and loop counters.  This file reads such a plan and launches it: it evaluates the
// polynomials for one call's arguments, fills the descriptors of include/tsb200.h and calls the
// family's entry point.  It is what the reference's generated C++ launcher (backend/driver.py:
// 102-246 of microsoft/triton-shared) needs in order to bind this library: the launcher keeps
// unmarshalling Python arguments and replaces its serial `for x, y, z` loop over the compiled
// kernel by one tsb_launch call.
//
// Nothing here allocates device memory: tables a launch needs on the device (the pid -> tile map
// of a matmul) are written into caller-provided scratch (tsb_launch_scratch_bytes).
#include "tsb_common.cuh"
#include <stdlib.h>
#include <string.h>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <utility>
#include <vector>

namespace tsb {
namespace plan {

// ---------------------------------------------------------------------------- JSON
struct Json {
  enum Type { NUL, BOOL, NUM, STR, ARR, OBJ } t = NUL;
  bool b = false;
  bool is_int = false;
  long long i = 0;
  double d = 0;
  std::string s;
  std::vector<Json> a;
  std::vector<std::pair<std::string, Json>> o;

  const Json *get(const char *key) const {
    for (auto &kv : o)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool is_null() const { return t == NUL; }
};

struct Parser {
  const char *p, *end;
  std::string err;
  explicit Parser(const char *s, size_t n) : p(s), end(s + n) {}
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p;
  }
  bool fail(const char *m) {
    if (err.empty()) err = m;
    return false;
  }
  bool value(Json &out, int depth = 0) {
    if (depth > 200) return fail("nesting too deep");
    ws();
    if (p >= end) return fail("unexpected end");
    if (*p == '{') {
      ++p;
      out.t = Json::OBJ;
      ws();
      if (p < end && *p == '}') { ++p; return true; }
      while (true) {
        Json k;
        ws();
        if (!string(k)) return false;
        ws();
        if (p >= end || *p != ':') return fail("expected ':'");
        ++p;
        Json v;
        if (!value(v, depth + 1)) return false;
        out.o.emplace_back(k.s, std::move(v));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == '}') { ++p; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (*p == '[') {
      ++p;
      out.t = Json::ARR;
      ws();
      if (p < end && *p == ']') { ++p; return true; }
      while (true) {
        Json v;
        if (!value(v, depth + 1)) return false;
        out.a.push_back(std::move(v));
        ws();
        if (p < end && *p == ',') { ++p; continue; }
        if (p < end && *p == ']') { ++p; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (*p == '"') return string(out);
    if (end - p >= 4 && !strncmp(p, "true", 4)) { p += 4; out.t = Json::BOOL; out.b = true; return true; }
    if (end - p >= 5 && !strncmp(p, "false", 5)) { p += 5; out.t = Json::BOOL; out.b = false; return true; }
    if (end - p >= 4 && !strncmp(p, "null", 4)) { p += 4; out.t = Json::NUL; return true; }
    // number
    const char *q = p;
    bool integral = true;
    if (q < end && (*q == '-' || *q == '+')) ++q;
    while (q < end && ((*q >= '0' && *q <= '9') || *q == '.' || *q == 'e' || *q == 'E' || *q == '-' || *q == '+')) {
      if (*q == '.' || *q == 'e' || *q == 'E') integral = false;
      ++q;
    }
    if (q == p) return fail("unexpected character");
    std::string num(p, q);
    out.t = Json::NUM;
    out.is_int = integral;
    out.d = strtod(num.c_str(), nullptr);
    out.i = integral ? strtoll(num.c_str(), nullptr, 10) : (long long)out.d;
    p = q;
    return true;
  }
  bool string(Json &out) {
    if (p >= end || *p != '"') return fail("expected string");
    ++p;
    out.t = Json::STR;
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
          case 'n': out.s.push_back('\n'); break;
          case 't': out.s.push_back('\t'); break;
          case 'u': out.s.push_back('?'); p += 4; break;  // names are ASCII
          default: out.s.push_back(*p);
        }
        ++p;
      } else {
        out.s.push_back(*p++);
      }
    }
    if (p >= end) return fail("unterminated string");
    ++p;
    return true;
  }
};

// ---------------------------------------------------------------------------- polynomials
// Atoms: ["arg", i] | ["pid", axis] | ["np", axis] | ["it", loop id] | ["fn", name, poly, poly]
struct Poly;
struct Atom {
  enum Kind { ARG, PID, NP, IT, FN } kind;
  long long idx = 0;
  std::string fn;
  std::shared_ptr<Poly> a, b;
};
struct Term {
  std::vector<Atom> atoms;
  long long coef = 0;
};
struct Poly {
  std::vector<Term> terms;
};

struct Env {
  const long long *args = nullptr;  // integer value per kernel argument position (0 where none)
  int n_args = 0;
  long long pid[3] = {0, 0, 0};
  long long np[3] = {1, 1, 1};
  std::vector<std::pair<long long, long long>> it;  // loop id -> counter
  long long counter(long long id) const {
    for (auto &kv : it)
      if (kv.first == id) return kv.second;
    return 0;
  }
  void set_counter(long long id, long long v) {
    for (auto &kv : it)
      if (kv.first == id) { kv.second = v; return; }
    it.emplace_back(id, v);
  }
};

static long long fn_eval(const std::string &n, long long a, long long b, bool &ok) {
  if (n == "divsi" || n == "remsi") {
    if (b == 0) b = 1;
    long long q = (a < 0 ? -a : a) / (b < 0 ? -b : b);
    if ((a < 0) != (b < 0)) q = -q;
    return n == "divsi" ? q : a - q * b;
  }
  if (n == "ceildivsi") {
    if (b == 0) b = 1;
    // -((-a) // b) with floor division, clamped at 0 (trip count of scf.for)
    long long na = -a, fl = na / b;
    if ((na % b != 0) && ((na < 0) != (b < 0))) --fl;
    long long q = -fl;
    return q > 0 ? q : 0;
  }
  if (n == "minsi") return a < b ? a : b;
  if (n == "maxsi") return a > b ? a : b;
  if (n == "andi") return a & b;
  if (n == "ori") return a | b;
  if (n == "xori") return a ^ b;
  if (n == "shli") return a << b;
  if (n == "shrsi") return a >> b;
  if (n.compare(0, 4, "cmp_") == 0) {
    const std::string c = n.substr(4);
    if (c == "slt" || c == "ult") return a < b;
    if (c == "sle" || c == "ule") return a <= b;
    if (c == "sgt" || c == "ugt") return a > b;
    if (c == "sge" || c == "uge") return a >= b;
    if (c == "eq") return a == b;
    if (c == "ne") return a != b;
  }
  ok = false;
  return 0;
}

static long long eval(const Poly &p, const Env &e, bool &ok) {
  long long total = 0;
  for (const Term &t : p.terms) {
    long long v = t.coef;
    for (const Atom &a : t.atoms) {
      switch (a.kind) {
        case Atom::ARG: v *= (a.idx >= 0 && a.idx < e.n_args) ? e.args[a.idx] : (ok = false, 0); break;
        case Atom::PID: v *= e.pid[a.idx]; break;
        case Atom::NP: v *= e.np[a.idx]; break;
        case Atom::IT: v *= e.counter(a.idx); break;
        case Atom::FN: v *= fn_eval(a.fn, eval(*a.a, e, ok), eval(*a.b, e, ok), ok); break;
      }
    }
    total += v;
  }
  return total;
}

static bool depends_on(const Poly &p, Atom::Kind k) {
  for (const Term &t : p.terms)
    for (const Atom &a : t.atoms) {
      if (a.kind == k) return true;
      if (a.kind == Atom::FN && (depends_on(*a.a, k) || depends_on(*a.b, k))) return true;
    }
  return false;
}

// every loop counter at most linearly, never multiplied by another counter or inside a function
static bool affine_in_its(const Poly &p) {
  for (const Term &t : p.terms) {
    int deg = 0;
    for (const Atom &a : t.atoms) {
      if (a.kind == Atom::IT) ++deg;
      else if (a.kind == Atom::FN && (depends_on(*a.a, Atom::IT) || depends_on(*a.b, Atom::IT))) return false;
    }
    if (deg > 1) return false;
  }
  return true;
}

static bool parse_poly(const Json &j, Poly &out, std::string &err);

static bool parse_atom(const Json &j, Atom &a, std::string &err) {
  if (j.t != Json::ARR || j.a.empty() || j.a[0].t != Json::STR) { err = "malformed atom"; return false; }
  const std::string &k = j.a[0].s;
  if (k == "fn") {
    if (j.a.size() != 4) { err = "malformed fn atom"; return false; }
    a.kind = Atom::FN;
    a.fn = j.a[1].s;
    a.a = std::make_shared<Poly>();
    a.b = std::make_shared<Poly>();
    Json wa, wb;  // nested polynomials are stored bare (term lists)
    wa.t = wb.t = Json::OBJ;
    return parse_poly(j.a[2], *a.a, err) && parse_poly(j.a[3], *a.b, err);
  }
  if (j.a.size() < 2) { err = "malformed atom"; return false; }
  a.idx = j.a[1].i;
  if (k == "arg") a.kind = Atom::ARG;
  else if (k == "pid") a.kind = Atom::PID;
  else if (k == "np") a.kind = Atom::NP;
  else if (k == "it") a.kind = Atom::IT;
  else { err = "polynomial over unknown symbol '" + k + "'"; return false; }
  if ((a.kind == Atom::PID || a.kind == Atom::NP) && (a.idx < 0 || a.idx > 2)) { err = "grid axis out of range"; return false; }
  return true;
}

// accepts {"$poly": terms} and the bare term list (as nested inside fn atoms)
static bool parse_poly(const Json &j, Poly &out, std::string &err) {
  const Json *terms = &j;
  if (j.t == Json::OBJ) {
    terms = j.get("$poly");
    if (!terms) { err = "expected a polynomial"; return false; }
  }
  if (terms->t != Json::ARR) { err = "expected a polynomial"; return false; }
  for (const Json &tj : terms->a) {
    if (tj.t != Json::ARR || tj.a.size() != 2 || tj.a[0].t != Json::ARR) { err = "malformed polynomial term"; return false; }
    Term t;
    t.coef = tj.a[1].i;
    for (const Json &aj : tj.a[0].a) {
      Atom a;
      if (!parse_atom(aj, a, err)) return false;
      t.atoms.push_back(std::move(a));
    }
    out.terms.push_back(std::move(t));
  }
  return true;
}



// ---------------------------------------------------------------------------- name tables
static int dtype_of(const std::string &n) {
  static const std::map<std::string, int> m = {{"f32", TSB_F32}, {"f16", TSB_F16}, {"bf16", TSB_BF16}, {"i32", TSB_I32},
                                               {"i16", TSB_I16}, {"i8", TSB_I8},   {"i1", TSB_I1},     {"i64", TSB_I64},
                                               {"f64", TSB_F64}, {"u32", TSB_U32}, {"u16", TSB_U16},   {"u8", TSB_U8}};
  auto it = m.find(n);
  return it == m.end() ? -1 : it->second;
}
static int opcode_of(const std::string &n) {
  static const std::map<std::string, int> m = {
      {"load", TSB_OP_LOAD}, {"store", TSB_OP_STORE}, {"const", TSB_OP_CONST}, {"mov", TSB_OP_MOV},
      {"addf", TSB_OP_ADDF}, {"subf", TSB_OP_SUBF}, {"mulf", TSB_OP_MULF}, {"divf", TSB_OP_DIVF},
      {"maxnumf", TSB_OP_MAXNUMF}, {"minnumf", TSB_OP_MINNUMF}, {"maximumf", TSB_OP_MAXIMUMF},
      {"minimumf", TSB_OP_MINIMUMF}, {"remf", TSB_OP_REMF},
      {"exp", TSB_OP_EXP}, {"exp2", TSB_OP_EXP2}, {"log", TSB_OP_LOG}, {"log2", TSB_OP_LOG2}, {"sqrt", TSB_OP_SQRT},
      {"rsqrt", TSB_OP_RSQRT}, {"sin", TSB_OP_SIN}, {"cos", TSB_OP_COS}, {"tanh", TSB_OP_TANH}, {"erf", TSB_OP_ERF},
      {"absf", TSB_OP_ABSF}, {"negf", TSB_OP_NEGF}, {"floor", TSB_OP_FLOOR}, {"ceil", TSB_OP_CEIL},
      {"addi", TSB_OP_ADDI}, {"subi", TSB_OP_SUBI}, {"muli", TSB_OP_MULI}, {"divsi", TSB_OP_DIVSI},
      {"remsi", TSB_OP_REMSI}, {"divui", TSB_OP_DIVUI}, {"remui", TSB_OP_REMUI}, {"minsi", TSB_OP_MINSI},
      {"maxsi", TSB_OP_MAXSI}, {"minui", TSB_OP_MINUI}, {"maxui", TSB_OP_MAXUI}, {"andi", TSB_OP_ANDI},
      {"ori", TSB_OP_ORI}, {"xori", TSB_OP_XORI}, {"shli", TSB_OP_SHLI}, {"shrsi", TSB_OP_SHRSI},
      {"shrui", TSB_OP_SHRUI}, {"absi", TSB_OP_ABSI}, {"cmpf", TSB_OP_CMPF}, {"cmpi", TSB_OP_CMPI},
      {"select", TSB_OP_SELECT}, {"cast", TSB_OP_CAST}, {"bitcast", TSB_OP_BITCAST}, {"fma", TSB_OP_FMA},
      {"reduce", TSB_OP_REDUCE}, {"loop_begin", TSB_OP_LOOP_BEGIN}, {"loop_end", TSB_OP_LOOP_END},
      {"argreduce", TSB_OP_ARGREDUCE}, {"scan", TSB_OP_SCAN}};
  auto it = m.find(n);
  return it == m.end() ? -1 : it->second;
}

// ---------------------------------------------------------------------------- arguments of one call
struct Call {
  const int32_t *grid;
  long long pid_lo, pid_hi;
  void *stream;
  void *const *ptrs;
  const tsb_scalar *scalars;
  int n_args;
  void *scratch;
  long long scratch_bytes;
  int32_t *status;
  std::vector<long long> ints;  // integer value per argument position

  Env env() const {
    Env e;
    e.args = ints.data();
    e.n_args = n_args;
    for (int a = 0; a < 3; ++a) e.np[a] = grid[a];
    return e;
  }
  // what the launch parameters depend on: integer and float scalars and the grid
  std::string key() const {
    std::string k((const char *)grid, 3 * sizeof(int32_t));
    for (int i = 0; i < n_args; ++i) {
      k.append((const char *)&scalars[i].kind, sizeof(int32_t));
      k.append((const char *)&scalars[i].i, sizeof(int64_t));
      k.append((const char *)&scalars[i].f, sizeof(double));
    }
    return k;
  }
  char *pointer(long long arg) const { return (arg >= 0 && arg < n_args) ? (char *)ptrs[arg] : nullptr; }
};

struct Error {
  int code;
  std::string msg;
};
#define PLAN_FAIL(code_, ...)                         \
  do {                                                \
    char buf__[400];                                  \
    snprintf(buf__, sizeof(buf__), __VA_ARGS__);      \
    throw Error{code_, buf__};                        \
  } while (0)

static long long ev(const Poly &p, const Env &e) {
  bool ok = true;
  const long long v = eval(p, e, ok);
  if (!ok) PLAN_FAIL(TSB_ERR_INVALID, "a plan polynomial names an argument or function this launch cannot supply");
  return v;
}

// value at program (0,0,0) and the increment per grid axis (0 along axes of extent 1)
static void affine_pid(const Poly &p, Env e, const int32_t grid[3], long long &v0, long long inc[3]) {
  e.pid[0] = e.pid[1] = e.pid[2] = 0;
  v0 = ev(p, e);
  for (int a = 0; a < 3; ++a) {
    inc[a] = 0;
    if (grid[a] <= 1) continue;
    e.pid[a] = 1;
    inc[a] = ev(p, e) - v0;
    e.pid[a] = 0;
  }
}

static Poly poly_of(const Json &j, const char *what) {
  Poly p;
  std::string err;
  if (!parse_poly(j, p, err)) PLAN_FAIL(TSB_ERR_INVALID, "plan field %s: %s", what, err.c_str());
  return p;
}
static const Json &field(const Json &o, const char *key) {
  const Json *v = o.get(key);
  if (!v) PLAN_FAIL(TSB_ERR_INVALID, "plan lacks field '%s'", key);
  return *v;
}
static Poly poly_field(const Json &o, const char *key) { return poly_of(field(o, key), key); }
static long long int_field(const Json &o, const char *key) { return field(o, key).i; }
static bool has(const Json &o, const char *key) {
  const Json *v = o.get(key);
  return v && !v->is_null();
}

// ---------------------------------------------------------------------------- plan families
struct Family {
  virtual ~Family() {}
  virtual void launch(const Call &c) = 0;
  virtual long long scratch_bytes(const Call &) { return 0; }
};


// ---- a segment: one body of the elementwise VM or of a block program -------------------------
struct SegAccess {
  int kind = 0;  // is_store field: 0 load, 1 store, 2 mask probe, 3 index probe
  int dtype = 0;
  long long arg = -1;
  Poly offset;
  std::vector<Poly> strides;
  std::vector<bool> masked;
  std::vector<Poly> mstart, mbound;
  std::vector<Poly> conds;
  bool has_other = false;
  unsigned long long other = 0;
  struct W {
    int dim;
    Poly offset, stride, modulus, scale;
  };
  std::vector<W> wraps;
};
struct SegOp {
  int opcode, dtype, dst, a, b, c;
  // immediates: a number, a polynomial, a float argument, a loop trip count or (reductions) an opcode
  enum ImmKind { NUM, POLY, FARG, TRIP } kind[2] = {NUM, NUM};
  unsigned long long num[2] = {0, 0};
  Poly poly[2];
  long long ref[2] = {0, 0};  // argument position (FARG) or loop id (TRIP)
};
struct Segment {
  std::vector<int> space;
  std::vector<SegAccess> accs;
  std::vector<SegOp> ops;
  bool block_program = false;
  std::vector<std::pair<long long, int>> loop_depth;  // loop id -> nesting depth
};

static void parse_imm(const Json &j, SegOp &o, int k) {
  if (j.t == Json::NUM) {
    o.num[k] = (unsigned long long)j.i;
  } else if (j.t == Json::STR) {
    const int opc = opcode_of(j.s);
    if (opc < 0) PLAN_FAIL(TSB_ERR_INVALID, "unknown combiner '%s'", j.s.c_str());
    o.num[k] = (unsigned)opc;
  } else if (j.t == Json::ARR && j.a.size() == 2 && j.a[0].t == Json::STR) {
    const std::string &tag = j.a[0].s;
    if (tag == "poly") { o.kind[k] = SegOp::POLY; o.poly[k] = poly_of(j.a[1], "immediate"); }
    else if (tag == "farg") { o.kind[k] = SegOp::FARG; o.ref[k] = j.a[1].i; }
    else if (tag == "trip") { o.kind[k] = SegOp::TRIP; o.ref[k] = j.a[1].i; }
    else PLAN_FAIL(TSB_ERR_INVALID, "unknown immediate form '%s'", tag.c_str());
  } else if (!j.is_null()) {
    PLAN_FAIL(TSB_ERR_INVALID, "malformed immediate");
  }
}

static Segment parse_segment(const Json &j, bool block_program) {
  Segment sg;
  sg.block_program = block_program;
  for (const Json &d : field(j, "space").a) sg.space.push_back((int)d.i);
  const size_t rank = sg.space.size();
  for (const Json &d : field(j, "accs").a) {
    SegAccess a;
    const std::string &kind = field(d, "kind").s;
    a.kind = kind == "load" ? 0 : kind == "store" ? 1 : kind == "maskprobe" ? 2 : kind == "index" ? 3 : -1;
    a.dtype = dtype_of(field(d, "elem").s);
    if (a.kind < 0 || a.dtype < 0) PLAN_FAIL(TSB_ERR_INVALID, "access of unknown kind or element type");
    if (has(d, "arg")) a.arg = field(d, "arg").i;
    a.offset = poly_field(d, "offset");
    const Json &st = field(d, "strides"), &mk = field(d, "mask");
    if (st.a.size() != rank || mk.a.size() != rank) PLAN_FAIL(TSB_ERR_INVALID, "access rank differs from the iteration space");
    for (size_t k = 0; k < rank; ++k) {
      a.strides.push_back(poly_of(st.a[k], "strides"));
      const bool m = !mk.a[k].is_null();
      a.masked.push_back(m);
      a.mstart.push_back(m ? poly_of(mk.a[k].a.at(0), "mask") : Poly());
      a.mbound.push_back(m ? poly_of(mk.a[k].a.at(1), "mask") : Poly());
    }
    for (const Json &c : field(d, "conds").a) a.conds.push_back(poly_of(c, "conds"));
    if (has(d, "other")) { a.has_other = true; a.other = (unsigned long long)field(d, "other").i; }
    if (const Json *w = d.get("wrap"))
      for (const Json &wj : w->a)
        a.wraps.push_back({(int)int_field(wj, "dim"), poly_field(wj, "offset"), poly_field(wj, "stride"),
                           poly_field(wj, "modulus"), poly_field(wj, "scale")});
    if (a.wraps.size() > 2) PLAN_FAIL(TSB_ERR_INVALID, "more than two wrap-around terms");
    sg.accs.push_back(std::move(a));
  }
  for (const Json &oj : field(j, "ops").a) {
    if (oj.t != Json::ARR || oj.a.size() != 8) PLAN_FAIL(TSB_ERR_INVALID, "malformed op");
    SegOp o;
    o.opcode = opcode_of(oj.a[0].s);
    o.dtype = dtype_of(oj.a[1].s);
    if (o.opcode < 0 || o.dtype < 0) PLAN_FAIL(TSB_ERR_INVALID, "unknown opcode '%s' or type '%s'", oj.a[0].s.c_str(), oj.a[1].s.c_str());
    o.dst = (int)oj.a[2].i; o.a = (int)oj.a[3].i; o.b = (int)oj.a[4].i; o.c = (int)oj.a[5].i;
    parse_imm(oj.a[6], o, 0);
    parse_imm(oj.a[7], o, 1);
    sg.ops.push_back(std::move(o));
  }
  if (const Json *ld = j.get("loop_depth"))
    for (auto &kv : ld->o) sg.loop_depth.emplace_back(atoll(kv.first.c_str()), (int)kv.second.i);
  return sg;
}

// one evaluated launch of a segment: descriptors ready for tsb_elementwise / tsb_block_program
struct SegLaunch {
  std::vector<tsb_access> accs;
  std::vector<tsb_op> ops;
  std::vector<long long> arg_of;
};

static unsigned float_bits(double v) {
  const float f = (float)v;
  unsigned u;
  memcpy(&u, &f, 4);
  return u;
}

// `trips`: loop id -> trip count polynomial, for TRIP immediates
static SegLaunch evaluate_segment(const Segment &sg, const Call &c, Env env,
                                  const std::vector<std::pair<long long, Poly>> &trips) {
  SegLaunch L;
  const int rank = (int)sg.space.size();
  L.accs.resize(sg.accs.size());
  for (size_t ai = 0; ai < sg.accs.size(); ++ai) {
    const SegAccess &d = sg.accs[ai];
    tsb_access &a = L.accs[ai];
    memset(&a, 0, sizeof(a));
    a.dtype = d.dtype;
    a.rank = rank;
    a.is_store = d.kind;
    long long inc[3];
    long long off0;
    affine_pid(d.offset, env, c.grid, off0, inc);
    a.offset0 = off0;
    for (int k = 0; k < 3; ++k) a.offset_pid[k] = inc[k];
    bool gate = true;
    for (const Poly &q : d.conds) gate = gate && ev(q, env) != 0;
    for (int k = 0; k < rank; ++k) {
      a.sizes[k] = sg.space[k];
      a.strides[k] = ev(d.strides[k], env);
      if (d.masked[k]) {
        a.masked[k] = 1;
        long long s0, sinc[3];
        affine_pid(d.mstart[k], env, c.grid, s0, sinc);
        a.mask_start0[k] = s0;
        for (int j = 0; j < 3; ++j) a.mask_start_pid[k][j] = sinc[j];
        a.mask_bound[k] = ev(d.mbound[k], env);
      }
    }
    if (!gate) {  // a false scalar conjunct empties the block (MaskAnalysis.cpp:224-267)
      a.masked[0] = 1;
      a.mask_bound[0] = -(1ll << 62);
    }
    if (d.has_other) { a.has_other = 1; a.other_bits = d.other; }
    a.n_wrap = (int)d.wraps.size();
    for (size_t wi = 0; wi < d.wraps.size(); ++wi) {
      tsb_wrap &w = a.wrap[wi];
      w.dim = d.wraps[wi].dim;
      long long o0, oinc[3];
      affine_pid(d.wraps[wi].offset, env, c.grid, o0, oinc);
      w.offset0 = o0;
      for (int j = 0; j < 3; ++j) w.offset_pid[j] = oinc[j];
      w.stride = ev(d.wraps[wi].stride, env);
      w.modulus = ev(d.wraps[wi].modulus, env);
      w.scale = ev(d.wraps[wi].scale, env);
      if (w.modulus <= 0) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "wrap-around access with a non-positive modulus");
    }
    // advance per iteration of each enclosing device-side loop (offsets and mask starts are affine
    // in the counters: the difference between counter 1 and counter 0)
    for (auto &ld : sg.loop_depth) {
      bool dep = depends_on(d.offset, Atom::IT);
      for (int k = 0; k < rank && !dep; ++k) dep = d.masked[k] && depends_on(d.mstart[k], Atom::IT);
      if (!dep) continue;
      Env e1 = env;
      e1.set_counter(ld.first, 1);
      if (ld.second < 0 || ld.second >= TSB_MAX_LOOPS) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "loops nested too deeply");
      a.offset_loop[ld.second] += ev(d.offset, e1) - off0;
      for (int k = 0; k < rank; ++k)
        if (d.masked[k]) a.mask_start_loop[k][ld.second] += ev(d.mstart[k], e1) - a.mask_start0[k];
    }
    L.arg_of.push_back(d.arg);
  }
  L.ops.resize(sg.ops.size());
  for (size_t k = 0; k < sg.ops.size(); ++k) {
    const SegOp &o = sg.ops[k];
    tsb_op &x = L.ops[k];
    memset(&x, 0, sizeof(x));
    x.opcode = o.opcode;
    x.type = o.dtype;
    unsigned imm[2];
    for (int q = 0; q < 2; ++q) {
      switch (o.kind[q]) {
        case SegOp::NUM: imm[q] = (unsigned)o.num[q]; break;
        case SegOp::POLY: imm[q] = (unsigned)(ev(o.poly[q], env) & 0xffffffffll); break;
        case SegOp::FARG:
          if (o.ref[q] < 0 || o.ref[q] >= c.n_args) PLAN_FAIL(TSB_ERR_INVALID, "float argument %lld missing", o.ref[q]);
          imm[q] = float_bits(c.scalars[o.ref[q]].f);
          break;
        case SegOp::TRIP: {
          long long t = -1;
          for (auto &tp : trips)
            if (tp.first == o.ref[q]) t = ev(tp.second, env);
          if (t < 0) t = 0;
          imm[q] = (unsigned)t;
          break;
        }
      }
    }
    x.imm = imm[0];
    x.imm2 = imm[1];
    // a store names no result; its dst field carries the mask operand when the store is flagged
    const unsigned flags = sg.block_program ? x.imm2 : x.imm;
    const bool store_mask = o.opcode == TSB_OP_STORE && o.kind[sg.block_program ? 1 : 0] == SegOp::NUM && (flags & TSB_MEM_MASK);
    x.dst = (o.opcode != TSB_OP_STORE || store_mask) ? o.dst : 0;
    x.a = o.a; x.b = o.b; x.c = o.c;
  }
  return L;
}

static void bind_pointers(SegLaunch &L, const Call &c) {
  for (size_t i = 0; i < L.accs.size(); ++i)
    if (L.arg_of[i] >= 0) L.accs[i].base = c.pointer(L.arg_of[i]);
}


// ---- elementwise family -----------------------------------------------------------------------
struct TreeNode {
  bool is_seg = false;
  int seg = 0;
  long long loop_id = 0;
  Poly lb, ub, step;
  std::vector<TreeNode> children;
};

static std::vector<TreeNode> parse_tree(const Json &j) {
  std::vector<TreeNode> out;
  for (const Json &n : j.a) {
    TreeNode t;
    if (n.a.at(0).s == "seg") {
      t.is_seg = true;
      t.seg = (int)n.a.at(1).i;
    } else {
      t.loop_id = n.a.at(1).i;
      t.lb = poly_of(n.a.at(2), "lb");
      t.ub = poly_of(n.a.at(3), "ub");
      t.step = poly_of(n.a.at(4), "step");
      t.children = parse_tree(n.a.at(5));
    }
    out.push_back(std::move(t));
  }
  return out;
}

template <typename V>
struct Memo {  // evaluated launch parameters per (scalars, grid)
  std::map<std::string, V> m;
  std::mutex mu;
  template <typename F>
  V &get(const Call &c, F compute) {
    std::lock_guard<std::mutex> g(mu);
    const std::string k = c.key();
    auto it = m.find(k);
    if (it == m.end()) {
      if (m.size() > 64) m.clear();
      it = m.emplace(k, compute()).first;
    }
    return it->second;
  }
};

struct Elementwise : Family {
  std::vector<Segment> segments;
  std::vector<TreeNode> tree;
  // perfect nest: one segment inside loops whose iterations only shift offsets and mask starts
  bool nest = false;
  int nest_seg = 0;
  std::vector<const TreeNode *> nest_loops;
  Memo<std::vector<SegLaunch>> memo;

  explicit Elementwise(const Json &p) {
    for (const Json &sj : field(p, "segments").a) segments.push_back(parse_segment(sj, false));
    tree = parse_tree(field(p, "tree"));
    find_nest();
  }

  void find_nest() {
    const std::vector<TreeNode> *node = &tree;
    std::vector<const TreeNode *> loops;
    while (node->size() == 1 && !(*node)[0].is_seg) {
      loops.push_back(&(*node)[0]);
      node = &(*node)[0].children;
    }
    if (loops.empty() || loops.size() > TSB_MAX_LOOPS || node->size() != 1 || !(*node)[0].is_seg) return;
    for (const TreeNode *l : loops)
      if (depends_on(l->lb, Atom::IT) || depends_on(l->ub, Atom::IT) || depends_on(l->step, Atom::IT)) return;
    const Segment &sg = segments.at((*node)[0].seg);
    for (const SegAccess &d : sg.accs) {
      for (const Poly &q : d.strides) if (depends_on(q, Atom::IT)) return;
      for (size_t k = 0; k < d.masked.size(); ++k)
        if (d.masked[k] && (depends_on(d.mbound[k], Atom::IT) || !affine_in_its(d.mstart[k]))) return;
      for (const Poly &q : d.conds) if (depends_on(q, Atom::IT)) return;
      for (const SegAccess::W &w : d.wraps)
        if (depends_on(w.offset, Atom::IT) || depends_on(w.stride, Atom::IT) || depends_on(w.modulus, Atom::IT) ||
            depends_on(w.scale, Atom::IT))
          return;
      if (!affine_in_its(d.offset)) return;
    }
    for (const SegOp &o : sg.ops)
      for (int q = 0; q < 2; ++q)
        if (o.kind[q] == SegOp::POLY && depends_on(o.poly[q], Atom::IT)) return;
    nest = true;
    nest_seg = (*node)[0].seg;
    nest_loops = loops;
  }

  std::vector<SegLaunch> schedule(const Call &c) {
    std::vector<SegLaunch> out;
    Env env = c.env();
    if (nest) {
      Segment sg = segments[nest_seg];
      std::vector<std::pair<long long, Poly>> trips;
      std::vector<SegOp> head, tail;
      for (size_t depth = 0; depth < nest_loops.size(); ++depth) {
        const TreeNode *l = nest_loops[depth];
        if (ev(l->step, env) <= 0) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "loop with a non-positive step");
        sg.loop_depth.emplace_back(l->loop_id, (int)depth);
        SegOp b;
        b.opcode = TSB_OP_LOOP_BEGIN; b.dtype = TSB_I32; b.dst = -1; b.a = (int)depth; b.b = b.c = 0;
        b.kind[0] = SegOp::TRIP; b.ref[0] = l->loop_id;
        head.push_back(b);
        SegOp e;
        e.opcode = TSB_OP_LOOP_END; e.dtype = TSB_I32; e.dst = -1; e.a = (int)depth; e.b = e.c = 0;
        tail.insert(tail.begin(), e);
        // trip = ceildiv(ub - lb, step), evaluated directly
        env.set_counter(l->loop_id, 0);
      }
      // trip counts as constant polynomials of this call
      for (const TreeNode *l : nest_loops) {
        const long long lo = ev(l->lb, env), hi = ev(l->ub, env), st = ev(l->step, env);
        long long t = hi > lo ? (hi - lo + st - 1) / st : 0;
        Poly tp;
        Term term;
        term.coef = t;
        tp.terms.push_back(term);
        trips.emplace_back(l->loop_id, tp);
      }
      std::vector<SegOp> ops = head;
      ops.insert(ops.end(), sg.ops.begin(), sg.ops.end());
      ops.insert(ops.end(), tail.begin(), tail.end());
      sg.ops = ops;
      out.push_back(evaluate_segment(sg, c, env, trips));
      return out;
    }
    walk(tree, c, env, out);
    return out;
  }

  void walk(const std::vector<TreeNode> &nodes, const Call &c, Env &env, std::vector<SegLaunch> &out) {
    for (const TreeNode &n : nodes) {
      if (n.is_seg) {
        out.push_back(evaluate_segment(segments.at(n.seg), c, env, {}));
        continue;
      }
      const long long lo = ev(n.lb, env), hi = ev(n.ub, env), st = ev(n.step, env);
      if (st <= 0) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "loop with a non-positive step");
      const long long trips = hi > lo ? (hi - lo + st - 1) / st : 0;
      if ((long long)out.size() + trips > 4096)
        PLAN_FAIL(TSB_ERR_UNSUPPORTED, "elementwise family: more than 4096 launches for one kernel call");
      for (long long it = 0; it < trips; ++it) {
        env.set_counter(n.loop_id, it);
        walk(n.children, c, env, out);
      }
      env.set_counter(n.loop_id, 0);
    }
  }

  void launch(const Call &c) override {
    const std::vector<SegLaunch> &ls = memo.get(c, [&] { return schedule(c); });
    for (const SegLaunch &cached : ls) {
      SegLaunch L = cached;  // pointers are per call: the cached evaluation stays shareable between threads
      bind_pointers(L, c);
      const int rc = tsb_elementwise(L.accs.data(), (int)L.accs.size(), L.ops.data(), (int)L.ops.size(), c.grid, c.pid_lo,
                                     c.pid_hi, c.stream);
      if (rc) throw Error{rc, tsb_last_error()};
    }
  }
};

// ---- block programs -----------------------------------------------------------------------------
struct BlockProgram : Family {
  Segment seg;
  std::vector<int32_t> reg_masks;
  std::vector<std::pair<long long, Poly>> trips;
  std::vector<long long> loops;
  Memo<SegLaunch> memo;

  explicit BlockProgram(const Json &p) {
    seg = parse_segment(field(p, "seg"), true);
    for (const Json &m : field(p, "reg_masks").a) reg_masks.push_back((int32_t)m.i);
    if (const Json *t = p.get("trips"))
      for (auto &kv : t->o) trips.emplace_back(atoll(kv.first.c_str()), poly_of(kv.second, "trips"));
    if (const Json *l = field(p, "seg").get("loops"))
      for (const Json &x : l->a) loops.push_back(x.i);
  }
  void launch(const Call &c) override {
    SegLaunch L = memo.get(c, [&] {
      Env env = c.env();
      for (long long id : loops) env.set_counter(id, 0);
      return evaluate_segment(seg, c, env, trips);
    });
    bind_pointers(L, c);
    const int rc = tsb_block_program(L.accs.data(), (int)L.accs.size(), L.ops.data(), (int)L.ops.size(), reg_masks.data(),
                                     (int)reg_masks.size(), c.grid, c.pid_lo, c.pid_hi, c.stream);
    if (rc) throw Error{rc, tsb_last_error()};
  }
};


// ---- row kernels and reductions ------------------------------------------------------------------
static void need_1d_grid(const Call &c, const char *fam) {
  if ((long long)c.grid[1] * c.grid[2] != 1) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "%s family: expects a 1-D grid", fam);
}

struct Softmax : Family {
  long long in_arg, out_arg, block;
  Poly in_off, out_off, n_cols;
  explicit Softmax(const Json &p)
      : in_arg(int_field(p, "in_arg")), out_arg(int_field(p, "out_arg")), block(int_field(p, "block")),
        in_off(poly_field(p, "in_off")), out_off(poly_field(p, "out_off")), n_cols(poly_field(p, "n_cols")) {}
  void launch(const Call &c) override {
    need_1d_grid(c, "softmax");
    const Env e = c.env();
    long long i0, iinc[3], o0, oinc[3];
    affine_pid(in_off, e, c.grid, i0, iinc);
    affine_pid(out_off, e, c.grid, o0, oinc);
    const int rc = tsb_softmax_rows(c.pointer(in_arg) + 4 * i0, c.pointer(out_arg) + 4 * o0, TSB_F32, iinc[0], oinc[0],
                                    ev(n_cols, e), block, c.pid_lo, c.pid_hi, c.stream);
    if (rc) throw Error{rc, tsb_last_error()};
  }
};

struct LayerNorm : Family {
  long long x, y, w, b, mean = -1, rstd = -1, eps_arg;
  int dtype;
  Poly x_off, y_off, mean_off, rstd_off, n;
  explicit LayerNorm(const Json &p)
      : x(int_field(p, "x")), y(int_field(p, "y")), w(int_field(p, "w")), b(int_field(p, "b")),
        eps_arg(int_field(p, "eps_arg")), dtype(dtype_of(field(p, "elem").s)), x_off(poly_field(p, "x_off")),
        y_off(poly_field(p, "y_off")), n(poly_field(p, "n")) {
    if (has(p, "mean")) { mean = int_field(p, "mean"); mean_off = poly_field(p, "mean_off"); }
    if (has(p, "rstd")) { rstd = int_field(p, "rstd"); rstd_off = poly_field(p, "rstd_off"); }
  }
  void launch(const Call &c) override {
    need_1d_grid(c, "layernorm");
    const Env e = c.env();
    long long x0, xinc[3], y0, yinc[3];
    affine_pid(x_off, e, c.grid, x0, xinc);
    affine_pid(y_off, e, c.grid, y0, yinc);
    const int es = dtype_size(dtype);
    float *mp = nullptr, *rp = nullptr;
    const Poly *offs[2] = {&mean_off, &rstd_off};
    const long long args[2] = {mean, rstd};
    float **dst[2] = {&mp, &rp};
    for (int k = 0; k < 2; ++k) {
      if (args[k] < 0) continue;
      long long o0, oinc[3];
      affine_pid(*offs[k], e, c.grid, o0, oinc);
      if (c.grid[0] > 1 && oinc[0] != 1) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "layernorm family: mean/rstd must be stored at index row");
      *dst[k] = (float *)(c.pointer(args[k]) + 4 * o0);
    }
    if (eps_arg < 0 || eps_arg >= c.n_args) PLAN_FAIL(TSB_ERR_INVALID, "layernorm family: eps argument missing");
    const int rc = tsb_layernorm_fwd(c.pointer(x) + es * x0, c.pointer(y) + es * y0, c.pointer(w), c.pointer(b), mp, rp,
                                     dtype, xinc[0], yinc[0], ev(n, e), (float)c.scalars[eps_arg].f, c.pid_lo, c.pid_hi,
                                     c.stream);
    if (rc) throw Error{rc, tsb_last_error()};
  }
};

struct ReduceRows : Family {
  long long x, out, block_rows;
  Poly stride_keep, stride_red, x_off, out_off, n_valid, row_start, row_bound;
  bool bounded;
  explicit ReduceRows(const Json &p)
      : x(int_field(p, "x")), out(int_field(p, "out")), block_rows(int_field(p, "block_rows")),
        stride_keep(poly_field(p, "stride_keep")), stride_red(poly_field(p, "stride_red")), x_off(poly_field(p, "x_off")),
        out_off(poly_field(p, "out_off")), n_valid(poly_field(p, "n_valid")), bounded(has(p, "row_bound")) {
    if (bounded) { row_start = poly_field(p, "row_start"); row_bound = poly_field(p, "row_bound"); }
  }
  struct R {
    long long sk, sr, x0, o0, n_valid, row_lo, row_hi;
  };
  R resolve(const Call &c) {
    need_1d_grid(c, "reduce_rows");
    const Env e = c.env();
    R r;
    r.sk = ev(stride_keep, e);
    r.sr = ev(stride_red, e);
    long long xinc[3], oinc[3];
    affine_pid(x_off, e, c.grid, r.x0, xinc);
    affine_pid(out_off, e, c.grid, r.o0, oinc);
    if (c.grid[0] > 1 && (xinc[0] != block_rows * r.sk || oinc[0] != block_rows))
      PLAN_FAIL(TSB_ERR_UNSUPPORTED, "reduce_rows family: programs do not tile the rows contiguously");
    r.n_valid = ev(n_valid, e);
    if (r.n_valid < 0) r.n_valid = 0;
    long long total = (long long)c.grid[0] * block_rows;
    if (bounded) {
      long long s0, sinc[3];
      affine_pid(row_start, e, c.grid, s0, sinc);
      if (s0 != 0 || (c.grid[0] > 1 && sinc[0] != block_rows))
        PLAN_FAIL(TSB_ERR_UNSUPPORTED, "reduce_rows family: row mask does not start at pid*BLOCK");
      const long long rb = ev(row_bound, e);
      if (rb < total) total = rb;
    }
    r.row_lo = c.pid_lo * block_rows < total ? c.pid_lo * block_rows : total;
    r.row_hi = c.pid_hi * block_rows < total ? c.pid_hi * block_rows : total;
    return r;
  }
  long long scratch_bytes(const Call &c) override {
    const R r = resolve(c);
    return r.row_hi > r.row_lo ? tsb_reduce_rows_scratch_bytes(r.row_hi - r.row_lo, r.n_valid, r.sk, r.sr) : 0;
  }
  void launch(const Call &c) override {
    const R r = resolve(c);
    if (r.row_hi <= r.row_lo) return;
    const long long need = tsb_reduce_rows_scratch_bytes(r.row_hi - r.row_lo, r.n_valid, r.sk, r.sr);
    if (need > c.scratch_bytes) PLAN_FAIL(TSB_ERR_INVALID, "reduce_rows family: %lld bytes of scratch needed, %lld given", need, c.scratch_bytes);
    const int rc = tsb_reduce_rows((const float *)(c.pointer(x) + 4 * r.x0), (float *)(c.pointer(out) + 4 * r.o0), r.sk, r.sr,
                                   1, r.n_valid, r.row_lo, r.row_hi, need > 0 ? c.scratch : nullptr, c.stream);
    if (rc) throw Error{rc, tsb_last_error()};
  }
};

struct ReduceAll : Family {
  long long x, out;
  Poly x_off, out_off, stride, n;
  explicit ReduceAll(const Json &p)
      : x(int_field(p, "x")), out(int_field(p, "out")), x_off(poly_field(p, "x_off")), out_off(poly_field(p, "out_off")),
        stride(poly_field(p, "stride")), n(poly_field(p, "n")) {}
  void launch(const Call &c) override {
    if (c.pid_hi <= c.pid_lo) return;
    const Env e = c.env();
    long long cnt = ev(n, e);
    if (cnt < 0) cnt = 0;
    const int rc = tsb_reduce_all((const float *)(c.pointer(x) + 4 * ev(x_off, e)), (float *)(c.pointer(out) + 4 * ev(out_off, e)),
                                  cnt, ev(stride, e), c.stream);
    if (rc) throw Error{rc, tsb_last_error()};
  }
};


// ---- tt.dot ---------------------------------------------------------------------------------------
struct Gemm : Family {
  long long a, b, c;
  int dtype, BM, BN, BK;
  long long loop;
  Poly a_base, a_adv, b_base, b_adv, sam, sak, sbk, sbn, scm, scn, c_off, trip;
  struct Bound { bool on = false; Poly start, bound; };
  Bound ka, kb, am, bn, cm, cn, tail_ka, tail_kb;
  struct Wrap { bool on = false; Poly offset, stride, modulus, scale; };
  Wrap a_wrap, b_wrap;
  bool has_tail = false;
  Poly tail_a_off, tail_b_off;

  static Bound bound_of(const Json &p, const char *key) {
    Bound b;
    if (has(p, key)) {
      b.on = true;
      b.start = poly_of(field(p, key).a.at(0), key);
      b.bound = poly_of(field(p, key).a.at(1), key);
    }
    return b;
  }
  static Wrap wrap_of(const Json &p, const char *key) {
    Wrap w;
    if (has(p, key)) {
      const Json &j = field(p, key);
      w.on = true;
      w.offset = poly_of(j.a.at(0), key); w.stride = poly_of(j.a.at(1), key);
      w.modulus = poly_of(j.a.at(2), key); w.scale = poly_of(j.a.at(3), key);
    }
    return w;
  }
  explicit Gemm(const Json &p)
      : a(int_field(p, "a")), b(int_field(p, "b")), c(int_field(p, "c")), dtype(dtype_of(field(p, "elem").s)),
        BM((int)int_field(p, "BM")), BN((int)int_field(p, "BN")), BK((int)int_field(p, "BK")), loop(int_field(p, "loop")),
        a_base(poly_field(p, "a_base")), a_adv(poly_field(p, "a_adv")), b_base(poly_field(p, "b_base")),
        b_adv(poly_field(p, "b_adv")), sam(poly_field(p, "sam")), sak(poly_field(p, "sak")), sbk(poly_field(p, "sbk")),
        sbn(poly_field(p, "sbn")), scm(poly_field(p, "scm")), scn(poly_field(p, "scn")), c_off(poly_field(p, "c_off")),
        trip(poly_field(p, "trip")) {
    ka = bound_of(p, "ka"); kb = bound_of(p, "kb"); am = bound_of(p, "am"); bn = bound_of(p, "bn");
    cm = bound_of(p, "cm"); cn = bound_of(p, "cn");
    a_wrap = wrap_of(p, "a_wrap"); b_wrap = wrap_of(p, "b_wrap");
    if (has(p, "tail")) {
      const Json &t = field(p, "tail");
      has_tail = true;
      tail_a_off = poly_field(t, "a_off"); tail_b_off = poly_field(t, "b_off");
      tail_ka = bound_of(t, "ka"); tail_kb = bound_of(t, "kb");
    }
  }

  struct R {
    long long M, N, K, sam, sak, sbk, sbn, scm, scn, n_prog;
    std::vector<int32_t> tiles;  // (tile_m, tile_n) per program of the full grid
    // split of a program range into vertically adjacent pairs and the rest
    long long split_lo = -1, split_hi = -1;
    std::vector<int32_t> pairs, singles;
    bool no_pairs = false;
  };
  Memo<R> memo;

  R resolve(const Call &c) {
    R r;
    Env e = c.env();
    e.set_counter(loop, 0);  // masks and offsets are read at the first K step
    r.sam = ev(sam, e); r.sak = ev(sak, e); r.sbk = ev(sbk, e); r.sbn = ev(sbn, e); r.scm = ev(scm, e); r.scn = ev(scn, e);
    long long steps = ev(trip, e);
    long long K = -1;
    bool have_k = false;
    for (const Bound *kbnd : {&ka, &kb}) {
      if (!kbnd->on) continue;
      const long long k_here = ev(kbnd->bound, e) - ev(kbnd->start, e);
      if (have_k && K != k_here) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: A and B K-masks disagree");
      K = k_here;
      have_k = true;
    }
    const long long loop_steps = steps;
    if (has_tail) {
      const long long ks = ev(tail_ka.start, e);
      if (ks != steps * BK || ev(tail_kb.start, e) != ks || ev(tail_kb.bound, e) != ev(tail_ka.bound, e))
        PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: the peeled K step does not continue where the loop ends");
      K = ev(tail_ka.bound, e);
      have_k = true;
      if (!(ks < K && K <= ks + BK)) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: the peeled K step is not one block");
      ++steps;
    }
    if (!have_k) K = steps * BK;
    if (steps != (K + BK - 1) / BK && !(K <= 0 && steps == 0))
      PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: loop runs %lld steps but K=%lld, BLOCK_K=%d", steps, K, BK);
    const long long adv_a = ev(a_adv, e), adv_b = ev(b_adv, e);
    if (adv_a != BK * r.sak || adv_b != BK * r.sbk)
      PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: pointers do not advance by BLOCK_K per iteration");
    r.K = K;
    const long long gx = c.grid[0], gy = c.grid[1], gz = c.grid[2];
    r.n_prog = gx * gy * gz;
    r.tiles.resize((size_t)(2 * r.n_prog));
    long long M = cm.on ? ev(cm.bound, e) : -1, N = cn.on ? ev(cn.bound, e) : -1;
    long long max_row = -BM, max_col = -BN;
    if (!cm.on && !a_wrap.on && r.sam == 0) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: cannot derive tile rows (stride_am == 0)");
    if (!cn.on && !b_wrap.on && r.sbn == 0) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: cannot derive tile columns (stride_bn == 0)");
    std::vector<long long> abase((size_t)r.n_prog), bbase((size_t)r.n_prog), aw((size_t)r.n_prog), bw((size_t)r.n_prog);
    for (long long lin = 0; lin < r.n_prog; ++lin) {
      e.pid[0] = lin % gx; e.pid[1] = (lin / gx) % gy; e.pid[2] = lin / (gx * gy);
      const long long ab = ev(a_base, e), bb = ev(b_base, e);
      abase[lin] = ab; bbase[lin] = bb;
      if (a_wrap.on) aw[lin] = ev(a_wrap.offset, e);
      if (b_wrap.on) bw[lin] = ev(b_wrap.offset, e);
      const long long row0 = cm.on ? ev(cm.start, e) : (a_wrap.on ? aw[lin] : ab / r.sam);
      const long long col0 = cn.on ? ev(cn.start, e) : (b_wrap.on ? bw[lin] : bb / r.sbn);
      if (row0 % BM || col0 % BN || row0 < 0 || col0 < 0) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: tiles are not aligned to the block shape");
      if (ev(c_off, e) != row0 * r.scm + col0 * r.scn) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: store offsets do not match the tile indices");
      if (has_tail && (ev(tail_a_off, e) != ab + loop_steps * adv_a || ev(tail_b_off, e) != bb + loop_steps * adv_b))
        PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: the peeled K step does not address the next K block");
      r.tiles[2 * lin] = (int32_t)(row0 / BM);
      r.tiles[2 * lin + 1] = (int32_t)(col0 / BN);
      if (row0 > max_row) max_row = row0;
      if (col0 > max_col) max_col = col0;
    }
    if (M < 0) M = r.n_prog ? max_row + BM : 0;
    if (N < 0) N = r.n_prog ? max_col + BN : 0;
    e.pid[0] = e.pid[1] = e.pid[2] = 0;
    if (a_wrap.on && (ev(a_wrap.modulus, e) != M || ev(a_wrap.stride, e) != 1 || ev(a_wrap.scale, e) != r.sam))
      PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: A row wrap-around is not `%% M` of the tile rows");
    if (b_wrap.on && (ev(b_wrap.modulus, e) != N || ev(b_wrap.stride, e) != 1 || ev(b_wrap.scale, e) != r.sbn))
      PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: B column wrap-around is not `%% N` of the tile columns");
    for (long long lin = 0; lin < r.n_prog; ++lin) {
      const long long row0 = (long long)r.tiles[2 * lin] * BM, col0 = (long long)r.tiles[2 * lin + 1] * BN;
      if (a_wrap.on ? (aw[lin] != row0 || abase[lin] != 0) : (abase[lin] != row0 * r.sam))
        PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: A offsets do not match the tile rows");
      if (b_wrap.on ? (bw[lin] != col0 || bbase[lin] != 0) : (bbase[lin] != col0 * r.sbn))
        PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: B offsets do not match the tile columns");
    }
    if (am.on && ev(am.bound, e) != M) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: mask bound of A rows differs from the store bound");
    if (bn.on && ev(bn.bound, e) != N) PLAN_FAIL(TSB_ERR_UNSUPPORTED, "gemm family: mask bound of B columns differs from the store bound");
    r.M = M; r.N = N;
    return r;
  }

  static void pair_tiles(R &r, long long lo, long long hi) {
    r.pairs.clear();
    r.singles.clear();
    std::map<std::pair<int, int>, long long> index;
    for (long long i = lo; i < hi; ++i) index[{r.tiles[2 * i], r.tiles[2 * i + 1]}] = i;
    std::vector<char> used((size_t)(hi - lo), 0);
    for (long long i = lo; i < hi; ++i) {
      const int tm = r.tiles[2 * i], tn = r.tiles[2 * i + 1];
      auto it = index.find({tm + 1, tn});
      if (tm % 2 == 0 && it != index.end()) {
        r.pairs.push_back(tm);
        r.pairs.push_back(tn);
        used[i - lo] = used[it->second - lo] = 1;
      }
    }
    for (long long i = lo; i < hi; ++i)
      if (!used[i - lo]) { r.singles.push_back(r.tiles[2 * i]); r.singles.push_back(r.tiles[2 * i + 1]); }
    r.split_lo = lo;
    r.split_hi = hi;
  }

  // device tables live in the caller's scratch: [pairs | singles] or the full tile table
  long long scratch_bytes(const Call &c) override {
    const R &r = memo.get(c, [&] { return resolve(c); });
    return (long long)r.tiles.size() * (long long)sizeof(int32_t) + 256;
  }

  void launch(const Call &c) override {
    R &r = memo.get(c, [&] { return resolve(c); });
    const long long need = (long long)r.tiles.size() * (long long)sizeof(int32_t) + 256;
    if (!c.scratch || c.scratch_bytes < need) PLAN_FAIL(TSB_ERR_INVALID, "gemm family: %lld bytes of scratch needed, %lld given", need, c.scratch_bytes);
    cudaStream_t s = (cudaStream_t)c.stream;
    char *dev = (char *)c.scratch;
    int rc;
    if (BM == 128 && r.K > 0 && !r.no_pairs) {
      if (r.split_lo != c.pid_lo || r.split_hi != c.pid_hi) pair_tiles(r, c.pid_lo, c.pid_hi);
      if (!r.pairs.empty()) {
        const size_t pb = r.pairs.size() * sizeof(int32_t), sb = r.singles.size() * sizeof(int32_t);
        const size_t soff = (pb + 255) & ~(size_t)255;
        if (cudaMemcpyAsync(dev, r.pairs.data(), pb, cudaMemcpyHostToDevice, s) != cudaSuccess)
          PLAN_FAIL(TSB_ERR_CUDA, "gemm family: upload of the tile-pair table failed");
        rc = tsb_gemm_paired(c.pointer(a), c.pointer(b), c.pointer(this->c), dtype, r.M, r.N, r.K, r.sam, r.sak, r.sbk, r.sbn,
                             r.scm, r.scn, BM, BN, BK, (const int32_t *)dev, (long long)r.pairs.size() / 2, c.status, s);
        if (rc == TSB_ERR_UNSUPPORTED) {
          r.no_pairs = true;  // operands not eligible: the one-CTA entry decides (tensor or SIMT)
        } else {
          if (rc) throw Error{rc, tsb_last_error()};
          if (!r.singles.empty()) {
            if (cudaMemcpyAsync(dev + soff, r.singles.data(), sb, cudaMemcpyHostToDevice, s) != cudaSuccess)
              PLAN_FAIL(TSB_ERR_CUDA, "gemm family: upload of the tile table failed");
            rc = tsb_gemm(c.pointer(a), c.pointer(b), c.pointer(this->c), dtype, r.M, r.N, r.K, r.sam, r.sak, r.sbk, r.sbn, r.scm,
                          r.scn, BM, BN, BK, (const int32_t *)(dev + soff), (long long)r.singles.size() / 2, 0,
                          (long long)r.singles.size() / 2, c.status, s);
            if (rc) throw Error{rc, tsb_last_error()};
          }
          return;
        }
      }
    }
    if (cudaMemcpyAsync(dev, r.tiles.data(), r.tiles.size() * sizeof(int32_t), cudaMemcpyHostToDevice, s) != cudaSuccess)
      PLAN_FAIL(TSB_ERR_CUDA, "gemm family: upload of the tile table failed");
    rc = tsb_gemm(c.pointer(a), c.pointer(b), c.pointer(this->c), dtype, r.M, r.N, r.K, r.sam, r.sak, r.sbk, r.sbn, r.scm, r.scn,
                  BM, BN, BK, (const int32_t *)dev, r.n_prog, c.pid_lo, c.pid_hi, c.status, s);
    if (rc) throw Error{rc, tsb_last_error()};
  }
};

}  // namespace plan
}  // namespace tsb

struct tsb_plan {
  std::string family, name;
  std::unique_ptr<tsb::plan::Family> impl;
};

using namespace tsb;
using namespace tsb::plan;

extern "C" tsb_plan *tsb_plan_create(const char *json, int64_t length) {
  if (!json) {
    set_error("tsb_plan_create: null plan text");
    return nullptr;
  }
  if (length < 0) length = (int64_t)strlen(json);
  Parser ps(json, (size_t)length);
  Json root;
  if (!ps.value(root) || root.t != Json::OBJ) {
    set_error("tsb_plan_create: plan is not valid JSON (%s)", ps.err.c_str());
    return nullptr;
  }
  try {
    std::unique_ptr<tsb_plan> p(new tsb_plan);
    p->family = field(root, "family").s;
    p->name = field(root, "name").s;
    const Json &params = field(root, "params");
    if (p->family == "elementwise") p->impl.reset(new Elementwise(params));
    else if (p->family == "block_program") p->impl.reset(new BlockProgram(params));
    else if (p->family == "softmax") p->impl.reset(new Softmax(params));
    else if (p->family == "layernorm") p->impl.reset(new LayerNorm(params));
    else if (p->family == "reduce_rows") p->impl.reset(new ReduceRows(params));
    else if (p->family == "reduce_all") p->impl.reset(new ReduceAll(params));
    else if (p->family == "gemm") p->impl.reset(new Gemm(params));
    else PLAN_FAIL(TSB_ERR_UNSUPPORTED, "unknown kernel family '%s'", p->family.c_str());
    return p.release();
  } catch (const Error &e) {
    set_error("tsb_plan_create: %s", e.msg.c_str());
  } catch (const std::exception &e) {
    set_error("tsb_plan_create: malformed plan (%s)", e.what());
  }
  return nullptr;
}

extern "C" void tsb_plan_destroy(tsb_plan *plan) { delete plan; }

extern "C" const char *tsb_plan_family(const tsb_plan *plan) { return plan ? plan->family.c_str() : ""; }
extern "C" const char *tsb_plan_kernel_name(const tsb_plan *plan) { return plan ? plan->name.c_str() : ""; }

static int make_call(const tsb_plan *plan, const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, void *stream,
                     void *const *ptr_args, const tsb_scalar *scalar_args, int n_args, void *scratch,
                     int64_t scratch_bytes, int32_t *status, Call &c, const char *who) {
  if (!plan || !plan->impl) return fail(TSB_ERR_INVALID, "%s: null plan", who);
  if (!grid || n_args < 0 || (n_args > 0 && (!ptr_args || !scalar_args))) return fail(TSB_ERR_INVALID, "%s: null argument", who);
  const long long total = (long long)grid[0] * grid[1] * grid[2];
  if (grid[0] < 0 || grid[1] < 0 || grid[2] < 0 || pid_lo < 0 || pid_hi > total || pid_lo > pid_hi)
    return fail(TSB_ERR_INVALID, "%s: program range [%lld,%lld) outside grid of %lld", who, (long long)pid_lo, (long long)pid_hi, total);
  c.grid = grid; c.pid_lo = pid_lo; c.pid_hi = pid_hi; c.stream = stream; c.ptrs = ptr_args; c.scalars = scalar_args;
  c.n_args = n_args; c.scratch = scratch; c.scratch_bytes = scratch_bytes; c.status = status;
  c.ints.resize((size_t)n_args);
  for (int i = 0; i < n_args; ++i) c.ints[i] = scalar_args[i].kind == TSB_SCALAR_INT ? scalar_args[i].i : 0;
  return TSB_OK;
}

extern "C" int64_t tsb_launch_scratch_bytes(const tsb_plan *plan, const int32_t grid[3], int64_t pid_lo, int64_t pid_hi,
                                            const tsb_scalar *scalar_args, int n_args) {
  Call c;
  static void *const no_ptrs[64] = {nullptr};
  if (n_args > 64) return fail(TSB_ERR_UNSUPPORTED, "tsb_launch_scratch_bytes: more than 64 kernel arguments");
  int rc = make_call(plan, grid, pid_lo, pid_hi, nullptr, no_ptrs, scalar_args, n_args, nullptr, 0, nullptr, c,
                     "tsb_launch_scratch_bytes");
  if (rc) return rc;
  try {
    return plan->impl->scratch_bytes(c);
  } catch (const Error &e) {
    return fail(e.code, "tsb_launch_scratch_bytes[%s]: %s", plan->name.c_str(), e.msg.c_str());
  } catch (const std::exception &e) {
    return fail(TSB_ERR_INVALID, "tsb_launch_scratch_bytes[%s]: %s", plan->name.c_str(), e.what());
  }
}

extern "C" int tsb_launch(const tsb_plan *plan, const int32_t grid[3], int64_t pid_lo, int64_t pid_hi, void *stream,
                          void *const *ptr_args, const tsb_scalar *scalar_args, int n_args, void *scratch,
                          int64_t scratch_bytes, int32_t *status) {
  Call c;
  int rc = make_call(plan, grid, pid_lo, pid_hi, stream, ptr_args, scalar_args, n_args, scratch, scratch_bytes, status, c,
                     "tsb_launch");
  if (rc) return rc;
  if (pid_hi == pid_lo) return TSB_OK;
  try {
    plan->impl->launch(c);
    return TSB_OK;
  } catch (const Error &e) {
    // the family's entry point has already left its message when the failure came from there
    return fail(e.code, "tsb_launch[%s]: %s", plan->name.c_str(), e.msg.c_str());
  } catch (const std::exception &e) {
    return fail(TSB_ERR_INVALID, "tsb_launch[%s]: %s", plan->name.c_str(), e.what());
  }
}
