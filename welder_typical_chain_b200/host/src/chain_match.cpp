// Dataflow matcher behind the chain recogniser.  The function body is cut into top-level
// statements (SSA name, operation, ins/outs operands, indexing maps, iterator types and the
// scalar operations of a linalg.generic region); the matcher then walks BACKWARDS from the
// returned value and accepts only the exact producer/consumer structure of the chains this
// build compiles:
//
//   matmul_softmax       return <- [truncf] <- softmax(x) ; x <- {scale mulf, extf}* <- matmul(A', B') with a zero fill,
//                        A'/B' the function arguments or their arith.truncf roundings
//                        (mlir/matmul_softmax_chain.mlir:15-80, ..._f16_native.mlir:13-92, ..._named_softmax.mlir:11-18,
//                        backend/welder/mlir_pipeline/matmul_softmax_chain_f16_matmul.mlir:13-129 in the reference)
//   row_softmax          return <- softmax(X), X the only argument (backend/welder/mlir_pipeline/softmax_row_chain.mlir:10-75)
//   layernorm_variance   return <- broadcast(var); var = c2 * rowsum((A - mean)^2); mean = c1 * rowsum(A)
//                        (backend/welder/mlir_pipeline/layernorm_variance_chain.mlir:12-104)
//
// where softmax(x) is either linalg.softmax over the last dimension or the four generics
// max / exp(x - max) / sum / divide with the right operands.  Every linalg operation of the
// function must take part in the match: a chain with anything extra (a factor applied after
// the division, a non-zero matmul init, an added constant) is rejected, not silently
// compiled as the fixed kernel.  The reference hands the text to MLIR itself
// (compiler/ir/ChainCanonicalize.cpp:77-163), which compiles what is written.
#include "wtc_host.h"

#include <cmath>
#include <cstdlib>
#include <map>
#include <regex>
#include <set>
#include <sstream>

namespace wtc {
namespace ir {
namespace {

struct TType {
  std::vector<int64_t> dims;   // empty: a scalar
  std::string elem;
};

struct BodyOp {
  std::string result, op;
  std::vector<std::string> args;
  double cst = 0.0;
};

struct Stmt {
  std::string result, op;
  std::vector<std::string> ins, outs;
  std::vector<TType> inTypes, outTypes;
  double cst = 0.0;                                  // arith.constant
  std::vector<std::string> iterators;                // linalg.generic
  std::vector<std::vector<std::string>> mapResults;  // per operand: the result expressions of its indexing map
  int mapDims = 0;
  std::vector<std::string> blockArgs;
  std::vector<BodyOp> body;
  std::string yielded;
  int softmaxDim = -1;
  bool used = false;
};

std::string trim(const std::string &s) {
  const size_t a = s.find_first_not_of(" \t\n\r"), b = s.find_last_not_of(" \t\n\r");
  return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}

std::vector<std::string> splitTop(const std::string &s, char sep) {
  std::vector<std::string> out;
  int depth = 0;
  std::string cur;
  for (char c : s) {
    if (c == '<' || c == '(' || c == '[') ++depth;
    else if (c == '>' || c == ')' || c == ']') --depth;
    if (c == sep && depth == 0) { out.push_back(trim(cur)); cur.clear(); }
    else cur += c;
  }
  if (!trim(cur).empty()) out.push_back(trim(cur));
  return out;
}

bool parseType(const std::string &t, TType &out) {
  static const std::regex tre(R"(^tensor<((?:[0-9]+x)+)(f16|f32)>$)");
  std::smatch m;
  const std::string s = trim(t);
  out.dims.clear();
  if (s == "f16" || s == "f32") { out.elem = s; return true; }
  if (!std::regex_match(s, m, tre)) return false;
  const std::string dims = m[1].str();
  for (size_t pos = 0; pos < dims.size();) {
    const size_t x = dims.find('x', pos);
    out.dims.push_back(std::stoll(dims.substr(pos, x - pos)));
    pos = x + 1;
  }
  out.elem = m[2].str();
  return true;
}

// text of the bracketed group that starts at s[open]
std::string group(const std::string &s, size_t open, char o, char c, size_t *endOut = nullptr) {
  int depth = 0;
  for (size_t i = open; i < s.size(); ++i) {
    if (s[i] == o) ++depth;
    else if (s[i] == c && --depth == 0) { if (endOut) *endOut = i; return s.substr(open + 1, i - open - 1); }
  }
  if (endOut) *endOut = std::string::npos;
  return "";
}

// "%a, %b : T1, T2" -> names and types
bool parseOperands(const std::string &text, std::vector<std::string> &names, std::vector<TType> &types) {
  const size_t colon = text.find(':');
  if (colon == std::string::npos) return false;
  names = splitTop(text.substr(0, colon), ',');
  for (const std::string &t : splitTop(text.substr(colon + 1), ',')) {
    TType ty;
    if (!parseType(t, ty)) return false;
    types.push_back(ty);
  }
  return names.size() == types.size() && !names.empty();
}

bool parseStatement(const std::string &raw, Stmt &st, std::string &diag) {
  std::string flat = raw;
  for (char &c : flat) if (c == '\n' || c == '\t') c = ' ';
  flat = trim(flat);
  static const std::regex retRe(R"(^(?:func\.)?return\s+(%[\w.]+))");
  std::smatch m;
  if (std::regex_search(flat, m, retRe)) { st.op = "return"; st.ins = {m[1].str()}; return true; }
  static const std::regex headRe(R"(^(%[\w.]+)\s*=\s*([a-z_]+\.[a-z_.]+))");
  if (!std::regex_search(flat, m, headRe)) { diag = "unrecognised statement: " + flat.substr(0, 60); return false; }
  st.result = m[1].str();
  st.op = m[2].str();
  if (st.op == "arith.constant") {
    static const std::regex cRe(R"(arith\.constant\s+([-+0-9.]+(?:[eE][-+]?[0-9]+)?)\s*:\s*(f16|f32))");
    if (!std::regex_search(flat, m, cRe)) { diag = "unsupported constant: " + flat.substr(0, 60); return false; }
    st.cst = std::strtod(m[1].str().c_str(), nullptr);
    return true;
  }
  if (st.op == "tensor.empty") return true;
  const size_t insPos = flat.find("ins("), outsPos = flat.find("outs(");
  if (insPos == std::string::npos || outsPos == std::string::npos) { diag = st.op + " without ins(...) outs(...)"; return false; }
  size_t outsEnd = 0;
  if (!parseOperands(group(flat, insPos + 3, '(', ')'), st.ins, st.inTypes) ||
      !parseOperands(group(flat, outsPos + 4, '(', ')', &outsEnd), st.outs, st.outTypes)) {
    diag = "cannot parse the operands of " + st.result;
    return false;
  }
  if (st.op == "linalg.softmax") {
    static const std::regex dRe(R"(dimension\(\s*([0-9]+)\s*\))");
    if (!std::regex_search(flat, m, dRe)) { diag = "linalg.softmax without dimension(d)"; return false; }
    st.softmaxDim = std::stoi(m[1].str());
    return true;
  }
  if (st.op != "linalg.generic") return true;   // fill, matmul, batch_matmul: operands are all that matters
  // ---- attributes
  const size_t itPos = flat.find("iterator_types");
  if (itPos == std::string::npos) { diag = "linalg.generic without iterator_types"; return false; }
  const std::string its = group(flat, flat.find('[', itPos), '[', ']');
  for (const std::string &t : splitTop(its, ',')) st.iterators.push_back(t.find("reduction") != std::string::npos ? "reduction" : "parallel");
  static const std::regex mapRe(R"(affine_map<\(([^)]*)\)\s*->\s*\(([^)]*)\)>)");
  const std::string head = flat.substr(0, insPos);
  for (auto it = std::sregex_iterator(head.begin(), head.end(), mapRe); it != std::sregex_iterator(); ++it) {
    st.mapDims = static_cast<int>(splitTop((*it)[1].str(), ',').size());
    st.mapResults.push_back(splitTop((*it)[2].str(), ','));
  }
  if (st.mapResults.size() != st.ins.size() + st.outs.size()) { diag = "indexing_maps do not match the operands of " + st.result; return false; }
  // ---- region (kept with its line breaks: one scalar operation per line)
  const size_t regOpenFlat = flat.find('{', outsEnd);
  if (regOpenFlat == std::string::npos) { diag = "linalg.generic without a region"; return false; }
  // locate the same brace in the raw text: it is the first '{' after the outs(...) group
  const size_t rawOuts = raw.find("outs(");
  size_t rawOutsEnd = 0;
  group(raw, rawOuts + 4, '(', ')', &rawOutsEnd);
  const size_t regOpen = raw.find('{', rawOutsEnd);
  const std::string region = group(raw, regOpen, '{', '}');
  std::istringstream in(region);
  std::string line;
  static const std::regex bbRe(R"(\^bb0\s*\(([^)]*)\))");
  static const std::regex opRe(R"(^(%[\w.]+)\s*=\s*((?:arith|math)\.[a-z_]+)\s+(.*)$)");
  static const std::regex yRe(R"(^linalg\.yield\s+(%[\w.]+))");
  while (std::getline(in, line)) {
    line = trim(line);
    if (line.empty()) continue;
    if (std::regex_search(line, m, bbRe)) {
      for (const std::string &a : splitTop(m[1].str(), ',')) st.blockArgs.push_back(trim(a.substr(0, a.find(':'))));
      continue;
    }
    if (std::regex_search(line, m, yRe)) { st.yielded = m[1].str(); continue; }
    if (!std::regex_search(line, m, opRe)) { diag = "unsupported operation inside " + st.result + ": " + line.substr(0, 60); return false; }
    BodyOp bo;
    bo.result = m[1].str();
    bo.op = m[2].str();
    std::string rest = m[3].str();
    const size_t colon = rest.rfind(':');
    if (colon != std::string::npos) rest = rest.substr(0, colon);
    if (bo.op == "arith.constant") bo.cst = std::strtod(trim(rest).c_str(), nullptr);
    else {
      const size_t attr = rest.find(" fastmath");
      if (attr != std::string::npos) rest = rest.substr(0, attr);
      for (const std::string &a : splitTop(rest, ',')) bo.args.push_back(a);
    }
    st.body.push_back(bo);
  }
  if (st.blockArgs.size() != st.ins.size() + st.outs.size() || st.yielded.empty()) { diag = "malformed region in " + st.result; return false; }
  return true;
}

// ---- shape of a generic -------------------------------------------------------------------------
bool isIdentity(const Stmt &s, size_t operand) {
  const auto &r = s.mapResults[operand];
  if (static_cast<int>(r.size()) != s.mapDims) return false;
  for (size_t i = 0; i < r.size(); ++i) if (r[i] != "d" + std::to_string(i)) return false;
  return true;
}
bool isDropLast(const Stmt &s, size_t operand) {
  const auto &r = s.mapResults[operand];
  if (static_cast<int>(r.size()) != s.mapDims - 1) return false;
  for (size_t i = 0; i < r.size(); ++i) if (r[i] != "d" + std::to_string(i)) return false;
  return true;
}
bool allParallel(const Stmt &s) {
  for (const auto &i : s.iterators) if (i != "parallel") return false;
  return true;
}
bool lastIsReduction(const Stmt &s) {
  if (s.iterators.empty() || s.iterators.back() != "reduction") return false;
  for (size_t i = 0; i + 1 < s.iterators.size(); ++i) if (s.iterators[i] != "parallel") return false;
  return true;
}
bool isMaxOp(const std::string &op) { return op == "arith.maximumf" || op == "arith.maxnumf" || op == "arith.maxf"; }
bool sameSet(const std::vector<std::string> &a, const std::string &x, const std::string &y) {
  return a.size() == 2 && ((a[0] == x && a[1] == y) || (a[0] == y && a[1] == x));
}

struct Matcher {
  std::map<std::string, Stmt *> def;
  std::map<std::string, double> outerConst;
  std::vector<std::string> args;          // function argument names
  std::vector<TType> argTypes;
  std::string diag;

  Stmt *producer(const std::string &v, const char *what) {
    auto it = def.find(v);
    if (it == def.end()) { if (diag.empty()) diag = std::string("no producer found for ") + what + " (" + v + ")"; return nullptr; }
    return it->second;
  }
  bool fail(const std::string &m) { if (diag.empty()) diag = m; return false; }

  // value `v` = linalg.fill of constant c (into a tensor.empty)
  bool isFillOf(const std::string &v, double &c) {
    Stmt *f = producer(v, "an init tensor");
    if (!f || f->op != "linalg.fill" || f->ins.size() != 1) return false;
    auto it = outerConst.find(f->ins[0]);
    if (it == outerConst.end()) return false;
    c = it->second;
    f->used = true;
    return true;
  }
  // elementwise generic with one tensor input, identity maps and body  y = OP(in [, const]) ; yield y
  bool unary(Stmt *g, const std::string &op, double *factor = nullptr) {
    if (!g || g->op != "linalg.generic" || g->ins.size() != 1 || g->outs.size() != 1 || !allParallel(*g) ||
        !isIdentity(*g, 0) || !isIdentity(*g, 1))
      return false;
    const std::string &in = g->blockArgs[0];
    std::map<std::string, double> local;
    const BodyOp *last = nullptr;
    for (const BodyOp &b : g->body) {
      if (b.op == "arith.constant") { local[b.result] = b.cst; continue; }
      if (last) return false;   // one arithmetic operation only
      last = &b;
    }
    if (!last || last->op != op || g->yielded != last->result) return false;
    if (op == "arith.mulf") {
      if (last->args.size() != 2) return false;
      const std::string other = last->args[0] == in ? last->args[1] : (last->args[1] == in ? last->args[0] : "");
      if (other.empty()) return false;
      auto c = local.find(other);
      auto oc = outerConst.find(other);
      if (c != local.end()) *factor = c->second;
      else if (oc != outerConst.end()) *factor = oc->second;
      else return false;
      return true;
    }
    return last->args.size() == 1 && last->args[0] == in;
  }
  // row reduction generic: ins(x) outs(init); maps [identity, dropLast]; body acc' = OP(in, acc)
  bool rowReduce(Stmt *g, bool wantMax, std::string &input, double &init) {
    if (!g || g->op != "linalg.generic" || g->ins.size() != 1 || g->outs.size() != 1 || !lastIsReduction(*g) ||
        !isIdentity(*g, 0) || !isDropLast(*g, 1) || g->body.size() != 1)
      return false;
    const BodyOp &b = g->body[0];
    if (!(wantMax ? isMaxOp(b.op) : b.op == "arith.addf")) return false;
    if (!sameSet(b.args, g->blockArgs[0], g->blockArgs[1]) || g->yielded != b.result) return false;
    if (!isFillOf(g->outs[0], init)) return false;
    input = g->ins[0];
    return true;
  }

  // `v` = row softmax of `x` over the last dimension
  bool softmax(const std::string &v, std::string &x, bool &named, int rank) {
    Stmt *d = producer(v, "the softmax result");
    if (!d) return false;
    if (d->op == "linalg.softmax") {
      if (d->softmaxDim != rank - 1) return fail("linalg.softmax must reduce the last dimension (row softmax)");
      if (d->ins.size() != 1) return fail("linalg.softmax takes one input");
      named = true; d->used = true; x = d->ins[0];
      return true;
    }
    named = false;
    // divide: ins(e, s), maps [identity, dropLast, identity], body e / s
    if (d->op != "linalg.generic" || d->ins.size() != 2 || !allParallel(*d) || !isIdentity(*d, 0) || !isDropLast(*d, 1) ||
        !isIdentity(*d, 2) || d->body.size() != 1 || d->body[0].op != "arith.divf" || d->body[0].args.size() != 2 ||
        d->body[0].args[0] != d->blockArgs[0] || d->body[0].args[1] != d->blockArgs[1] || d->yielded != d->body[0].result)
      return fail("the chain must end in the division exp / row_sum (found something else producing " + v + ")");
    d->used = true;
    Stmt *e = producer(d->ins[0], "the exponentials");
    Stmt *s = producer(d->ins[1], "the row sums");
    if (!e || !s) return false;
    // sum: addf reduction of the SAME exponentials, from a zero init
    std::string sumIn; double sumInit = 1.0;
    if (!rowReduce(s, false, sumIn, sumInit) || sumIn != d->ins[0]) return fail("the divisor must be the row sum (arith.addf reduction) of the exponentials");
    if (sumInit != 0.0) return fail("the row sum must start from 0");
    s->used = true;
    // exp: ins(x, max), maps [identity, dropLast, identity], body exp(x - max)
    if (e->op != "linalg.generic" || e->ins.size() != 2 || !allParallel(*e) || !isIdentity(*e, 0) || !isDropLast(*e, 1) ||
        !isIdentity(*e, 2) || e->body.size() != 2 || e->body[0].op != "arith.subf" || e->body[0].args.size() != 2 ||
        e->body[0].args[0] != e->blockArgs[0] || e->body[0].args[1] != e->blockArgs[1] || e->body[1].op != "math.exp" ||
        e->body[1].args.size() != 1 || e->body[1].args[0] != e->body[0].result || e->yielded != e->body[1].result)
      return fail("the exponentials must be math.exp(x - row_max)");
    e->used = true;
    Stmt *mx = producer(e->ins[1], "the row maxima");
    std::string maxIn; double maxInit = 0.0;
    if (!rowReduce(mx, true, maxIn, maxInit) || maxIn != e->ins[0]) return fail("the subtrahend must be the row maximum (arith.maximumf reduction) of the same values");
    if (!(maxInit <= -6.5e4)) return fail("the row maximum must start from the most negative value");
    mx->used = true;
    x = e->ins[0];
    return true;
  }

  int argIndex(const std::string &v) const {
    for (size_t i = 0; i < args.size(); ++i) if (args[i] == v) return static_cast<int>(i);
    return -1;
  }
};

} // namespace

bool matchChain(const std::string &text, ChainSpec &spec, std::string &diag) {
  // ---- function signature
  static const std::regex fnRe(R"(func\.func\s+@([A-Za-z_][\w]*)\s*\()");
  std::smatch fm;
  if (!std::regex_search(text, fm, fnRe)) { diag = "no func.func found"; return false; }
  spec.funcName = fm[1].str();
  const size_t open = static_cast<size_t>(fm.position(0) + fm.length(0) - 1);
  size_t sigEnd = 0;
  const std::string sig = group(text, open, '(', ')', &sigEnd);
  Matcher mt;
  for (const std::string &a : splitTop(sig, ',')) {
    const size_t colon = a.find(':');
    TType t;
    if (colon == std::string::npos || !parseType(a.substr(colon + 1), t) || t.dims.empty()) { diag = "function arguments must be static f16/f32 tensors"; return false; }
    mt.args.push_back(trim(a.substr(0, colon)));
    mt.argTypes.push_back(t);
  }
  const size_t bodyOpen = text.find('{', sigEnd);
  TType resType;
  {
    const size_t arrow = text.find("->", sigEnd);
    if (arrow == std::string::npos || bodyOpen == std::string::npos || arrow > bodyOpen || !parseType(text.substr(arrow + 2, bodyOpen - arrow - 2), resType) || resType.dims.empty()) {
      diag = "function result must be a static f16/f32 tensor";
      return false;
    }
  }
  const std::string body = group(text, bodyOpen, '{', '}');

  // ---- statements: a new one starts at brace depth 0 with "%name =" or "return"
  std::vector<std::string> chunks;
  {
    static const std::regex startRe(R"(^\s*(?:%[\w.]+\s*=|(?:func\.)?return\b))");
    std::istringstream in(body);
    std::string line, cur;
    int depth = 0;
    while (std::getline(in, line)) {
      if (depth == 0 && std::regex_search(line, startRe)) {
        if (!trim(cur).empty()) chunks.push_back(cur);
        cur.clear();
      }
      cur += line + "\n";
      for (char c : line) { if (c == '{') ++depth; else if (c == '}') --depth; }
    }
    if (!trim(cur).empty()) chunks.push_back(cur);
  }
  std::vector<Stmt> stmts(chunks.size());
  Stmt *ret = nullptr;
  for (size_t i = 0; i < chunks.size(); ++i) {
    if (!parseStatement(chunks[i], stmts[i], diag)) return false;
    if (stmts[i].op == "return") ret = &stmts[i];
    else {
      if (mt.def.count(stmts[i].result)) { diag = "value defined twice: " + stmts[i].result; return false; }
      mt.def[stmts[i].result] = &stmts[i];
      if (stmts[i].op == "arith.constant") mt.outerConst[stmts[i].result] = stmts[i].cst;
    }
  }
  if (!ret) { diag = "function has no return"; return false; }

  spec.matmulCount = countContains(text, "linalg.matmul") + countContains(text, "linalg.batch_matmul");
  spec.genericCount = countContains(text, "linalg.generic");
  spec.reductionCount = countContains(text, "\"reduction\"");
  spec.expCount = countContains(text, "math.exp");
  spec.divCount = countContains(text, "arith.divf");
  spec.outType = resType.elem;
  const int rank = static_cast<int>(resType.dims.size());

  auto finish = [&](bool ok) {
    if (!ok) { diag = mt.diag.empty() ? "the function is not one of the chains this build compiles" : mt.diag; return false; }
    for (const Stmt &s : stmts)
      if (!s.used && (s.op.rfind("linalg.", 0) == 0)) { diag = "operation outside the chain: " + s.result + " = " + s.op + " (every linalg operation must take part in the chain)"; return false; }
    diag.clear();
    return true;
  };

  std::string cur = ret->ins[0];
  // ---- layernorm variance chain: broadcast of a per-row value
  if (mt.args.size() == 1) {
    Stmt *last = mt.producer(cur, "the returned value");
    if (!last) return finish(false);
    if (last->op == "linalg.generic" && last->ins.size() == 1 && last->body.empty() && last->yielded == last->blockArgs[0] &&
        allParallel(*last) && isDropLast(*last, 0) && isIdentity(*last, 1)) {
      last->used = true;
      double c2 = 1.0, c1 = 1.0, i0 = 1.0, i1 = 1.0;
      Stmt *var = mt.producer(last->ins[0], "the variance");
      if (!mt.unary(var, "arith.mulf", &c2)) return finish(mt.fail("the broadcast value must be a row sum times a constant"));
      var->used = true;
      Stmt *sumsq = mt.producer(var->ins[0], "the sum of squares");
      std::string sqv;
      if (!mt.rowReduce(sumsq, false, sqv, i0) || i0 != 0.0) return finish(mt.fail("the variance must come from an arith.addf row reduction starting at 0"));
      sumsq->used = true;
      Stmt *sq = mt.producer(sqv, "the squared differences");
      if (!sq || sq->op != "linalg.generic" || sq->ins.size() != 2 || !allParallel(*sq) || !isIdentity(*sq, 0) || !isDropLast(*sq, 1) ||
          !isIdentity(*sq, 2) || sq->body.size() != 2 || sq->body[0].op != "arith.subf" || sq->body[0].args.size() != 2 ||
          sq->body[0].args[0] != sq->blockArgs[0] || sq->body[0].args[1] != sq->blockArgs[1] || sq->body[1].op != "arith.mulf" ||
          !sameSet(sq->body[1].args, sq->body[0].result, sq->body[0].result) || sq->yielded != sq->body[1].result)
        return finish(mt.fail("the reduced values must be (a - mean)^2"));
      sq->used = true;
      if (mt.argIndex(sq->ins[0]) != 0) return finish(mt.fail("(a - mean)^2 must read the function argument"));
      Stmt *mean = mt.producer(sq->ins[1], "the mean");
      if (!mt.unary(mean, "arith.mulf", &c1)) return finish(mt.fail("the mean must be a row sum times a constant"));
      mean->used = true;
      Stmt *sum = mt.producer(mean->ins[0], "the row sum");
      std::string sumIn;
      if (!mt.rowReduce(sum, false, sumIn, i1) || i1 != 0.0 || mt.argIndex(sumIn) != 0) return finish(mt.fail("the mean must come from an arith.addf row reduction of the argument"));
      sum->used = true;
      if (mt.argTypes[0].dims.size() != 2 || resType.dims != mt.argTypes[0].dims) return finish(mt.fail("layernorm variance chain: a 2-D argument and a result of the same shape"));
      spec.kind = "layernorm_variance";
      spec.M = mt.argTypes[0].dims[0]; spec.N = mt.argTypes[0].dims[1]; spec.K = 0; spec.batch = 1;
      spec.inType = spec.argType = spec.accType = mt.argTypes[0].elem;
      spec.meanFactor = c1; spec.varFactor = c2;
      return finish(true);
    }
    // ---- row softmax of the argument
    std::string x; bool named = false;
    if (!mt.softmax(cur, x, named, rank)) return finish(false);
    if (mt.argIndex(x) != 0) return finish(mt.fail("row softmax chain: the softmax must read the function argument"));
    if (resType.dims != mt.argTypes[0].dims) return finish(mt.fail("row softmax chain: result shape must equal the argument's"));
    spec.kind = "row_softmax";
    spec.namedSoftmax = named;
    const auto &d = mt.argTypes[0].dims;
    spec.N = d.back(); spec.M = 1;
    for (size_t i = 0; i + 1 < d.size(); ++i) spec.M *= d[i];
    spec.K = 0; spec.batch = 1;
    spec.inType = spec.argType = spec.accType = mt.argTypes[0].elem;
    return finish(true);
  }

  // ---- matmul -> softmax
  if (mt.args.size() != 2) { diag = "expected two tensor arguments (A, B), or one for the row-only chains; found " + std::to_string(mt.args.size()); return false; }
  spec.kind = "matmul_softmax";
  if (spec.matmulCount == 0) { diag = "no linalg.matmul / linalg.batch_matmul in the chain"; return false; }
  Stmt *tail = mt.producer(cur, "the returned value");
  if (!tail) return finish(false);
  if (mt.unary(tail, "arith.truncf")) { tail->used = true; cur = tail->ins[0]; }   // f32 probabilities rounded to the f16 result
  std::string x; bool named = false;
  if (!mt.softmax(cur, x, named, rank)) return finish(false);
  spec.namedSoftmax = named;
  // between the matmul and the softmax: constant factors and the widening of an f16 result
  Stmt *mm = nullptr;
  for (int guard = 0; guard < 8; ++guard) {
    Stmt *p = mt.producer(x, "the softmax input");
    if (!p) return finish(false);
    double f = 1.0;
    if (p->op == "linalg.matmul" || p->op == "linalg.batch_matmul") { mm = p; break; }
    if (mt.unary(p, "arith.mulf", &f)) { spec.scale *= f; p->used = true; x = p->ins[0]; continue; }
    if (mt.unary(p, "arith.extf")) { p->used = true; x = p->ins[0]; continue; }
    return finish(mt.fail("between the matmul and the softmax only a constant factor (arith.mulf) and arith.extf are accepted; found " + p->result + " = " + p->op));
  }
  if (!mm) return finish(mt.fail("no matmul feeds the softmax"));
  mm->used = true;
  spec.batched = mm->op == "linalg.batch_matmul";
  const size_t mrank = spec.batched ? 3 : 2;
  if (mm->ins.size() != 2 || mm->outs.size() != 1) return finish(mt.fail("matmul needs two inputs and one output tensor"));
  const TType &a = mm->inTypes[0], &b = mm->inTypes[1], &c = mm->outTypes[0];
  if (a.dims.size() != mrank || b.dims.size() != mrank || c.dims.size() != mrank) return finish(mt.fail("matmul operand ranks do not match the op"));
  const size_t o = spec.batched ? 1 : 0;
  spec.batch = spec.batched ? a.dims[0] : 1;
  spec.bBatched = spec.batched;
  spec.M = a.dims[o]; spec.K = a.dims[o + 1]; spec.N = b.dims[o + 1];
  if (b.dims[o] != spec.K) return finish(mt.fail("K mismatch between A and B"));
  if (c.dims[o] != spec.M || c.dims[o + 1] != spec.N || (spec.batched && (b.dims[0] != spec.batch || c.dims[0] != spec.batch)))
    return finish(mt.fail("matmul result shape does not match its operands"));
  if (a.elem != b.elem) return finish(mt.fail("A and B must share an element type"));
  if (resType.dims != c.dims) return finish(mt.fail("function result shape must equal the matmul result shape"));
  double init = 1.0;
  if (!mt.isFillOf(mm->outs[0], init)) return finish(mt.fail("the matmul must accumulate into a linalg.fill of a constant"));
  if (init != 0.0) return finish(mt.fail("the matmul must start from a zero fill (found a non-zero init)"));
  // operands: the function arguments, or their roundings to f16
  for (int k = 0; k < 2; ++k) {
    std::string v = mm->ins[k];
    if (mt.argIndex(v) < 0) {
      Stmt *t = mt.producer(v, k == 0 ? "the matmul's A operand" : "the matmul's B operand");
      if (!mt.unary(t, "arith.truncf")) return finish(mt.fail("matmul must consume the function arguments directly, or f32 arguments rounded to f16 by arith.truncf"));
      t->used = true;
      v = t->ins[0];
    }
    if (mt.argIndex(v) != k) return finish(mt.fail("the matmul's operands must be the function's first and second argument, in that order"));
    if (mt.argTypes[k].dims != mm->inTypes[k].dims) return finish(mt.fail("matmul must consume the function arguments (shapes differ)"));
  }
  if (mt.argTypes[0].elem != mt.argTypes[1].elem) return finish(mt.fail("A and B arguments must share an element type"));
  if (a.elem != mt.argTypes[0].elem && !(mt.argTypes[0].elem == "f32" && a.elem == "f16"))
    return finish(mt.fail("only the rounding f32 -> f16 is accepted between the arguments and the matmul"));
  spec.argType = mt.argTypes[0].elem;
  spec.inType = a.elem;
  spec.accType = c.elem;
  if (spec.matmulCount != 1) return finish(mt.fail("expected exactly one matmul in the chain"));
  return finish(true);
}

} // namespace ir
} // namespace wtc
