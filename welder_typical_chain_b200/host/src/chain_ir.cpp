// Chain recogniser for the one operator this build serves:
//   func @main(%A: tensor<[b x] M x K x T>, %B: tensor<[b x] K x N x T>) -> tensor<[b x] M x N x U>
//   [two generics arith.truncf f32 -> f16 on %A and %B]
//   linalg.matmul | linalg.batch_matmul  ins(%A, %B) outs(<fill 0> : tensor<.. x Tacc>)
//   [generic extf] [generic arith.mulf by a constant = scale]
//   either  linalg.softmax dimension(last)
//   or      generics  max (arith.maximumf|maxnumf|maxf, "reduction"), exp(x - max), sum (arith.addf,
//           "reduction"), x / sum        (mlir/matmul_softmax_chain.mlir:15-80 in the reference)
//   [generic arith.truncf]
// The reference hands this text to mlir-opt (compiler/ir/ChainCanonicalize.cpp:77-163); here a
// text recogniser extracts shapes, element types and the scale, and rewrites linalg.softmax into
// the four generics itself.
#include "wtc_host.h"

#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <map>
#include <regex>
#include <sstream>

namespace wtc {

std::string readAll(const std::string &path) {
  std::ifstream ifs(path);
  if (!ifs) return "";
  std::ostringstream oss;
  oss << ifs.rdbuf();
  return oss.str();
}

bool writeAll(const std::string &path, const std::string &content) {
  std::error_code ec;
  const auto parent = std::filesystem::path(path).parent_path();
  if (!parent.empty()) std::filesystem::create_directories(parent, ec);
  std::ofstream ofs(path);
  if (!ofs) return false;
  ofs << content;
  return static_cast<bool>(ofs);
}

int countContains(const std::string &text, const std::string &needle) {
  if (needle.empty()) return 0;
  int n = 0;
  for (size_t pos = text.find(needle); pos != std::string::npos; pos = text.find(needle, pos + needle.size())) ++n;
  return n;
}

namespace ir {
namespace {

struct TensorType {
  std::vector<int64_t> dims;
  std::string elem;
};

std::string stripComments(const std::string &text) {
  std::ostringstream out;
  std::istringstream in(text);
  std::string line;
  while (std::getline(in, line)) {
    const size_t p = line.find("//");
    out << (p == std::string::npos ? line : line.substr(0, p)) << '\n';
  }
  return out.str();
}

// Attribute and type aliases (`#map = affine_map<...>`, `!row_t = tensor<...>`), which MLIR
// printers emit at the top of a module, are expanded in place so that the rest of the
// recogniser only ever sees spelled-out types.  Definitions may use earlier aliases.
std::string expandAliases(const std::string &text) {
  static const std::regex defRe(R"(^[ \t]*([#!][A-Za-z_][\w.$-]*)[ \t]*=[ \t]*(.*\S)[ \t]*$)");
  std::vector<std::pair<std::string, std::string>> defs;
  std::ostringstream body;
  std::istringstream in(text);
  std::string line;
  bool top = true;
  while (std::getline(in, line)) {
    if (top) {
      const size_t c = line.find("//");
      const std::string code = c == std::string::npos ? line : line.substr(0, c);
      std::smatch m;
      if (std::regex_match(code, m, defRe)) { defs.emplace_back(m[1].str(), m[2].str()); continue; }
      if (code.find("module") != std::string::npos || code.find("func.func") != std::string::npos) top = false;
    }
    body << line << '\n';
  }
  if (defs.empty()) return text;
  auto substitute = [&](std::string s) {
    for (int pass = 0; pass < 4; ++pass) {
      bool changed = false;
      for (const auto &d : defs) {
        size_t pos = 0;
        while ((pos = s.find(d.first, pos)) != std::string::npos) {
          const size_t end = pos + d.first.size();
          const bool boundary = end >= s.size() || !(std::isalnum(static_cast<unsigned char>(s[end])) || s[end] == '_' || s[end] == '.' || s[end] == '$' || s[end] == '-');
          if (!boundary) { pos = end; continue; }
          s.replace(pos, d.first.size(), d.second);
          pos += d.second.size();
          changed = true;
        }
      }
      if (!changed) break;
    }
    return s;
  };
  return substitute(body.str());
}

bool parseTensorType(const std::string &s, TensorType &t) {
  static const std::regex re(R"(tensor<((?:[0-9]+x)+)(f16|f32)>)");
  std::smatch m;
  if (!std::regex_search(s, m, re)) return false;
  t.dims.clear();
  std::string dims = m[1].str();
  size_t pos = 0;
  while (pos < dims.size()) {
    const size_t x = dims.find('x', pos);
    t.dims.push_back(std::stoll(dims.substr(pos, x - pos)));
    pos = x + 1;
  }
  t.elem = m[2].str();
  return true;
}

std::vector<TensorType> allTensorTypes(const std::string &s) {
  std::vector<TensorType> out;
  static const std::regex re(R"(tensor<(?:[0-9]+x)+(?:f16|f32)>)");
  for (auto it = std::sregex_iterator(s.begin(), s.end(), re); it != std::sregex_iterator(); ++it) {
    TensorType t;
    if (parseTensorType(it->str(), t)) out.push_back(t);
  }
  return out;
}

// text of the parenthesised group that starts at s[open] == '('
std::string parenGroup(const std::string &s, size_t open) {
  int depth = 0;
  for (size_t i = open; i < s.size(); ++i) {
    if (s[i] == '(') ++depth;
    else if (s[i] == ')' && --depth == 0) return s.substr(open + 1, i - open - 1);
  }
  return "";
}

std::string typeStr(const std::vector<int64_t> &dims, const std::string &elem) {
  std::string s = "tensor<";
  for (int64_t d : dims) s += std::to_string(d) + "x";
  return s + elem + ">";
}

std::string identityMap(int rank) {
  std::string d;
  for (int i = 0; i < rank; ++i) d += (i ? ", d" : "d") + std::to_string(i);
  return "affine_map<(" + d + ") -> (" + d + ")>";
}
std::string dropLastMap(int rank) {
  std::string d, r;
  for (int i = 0; i < rank; ++i) d += (i ? ", d" : "d") + std::to_string(i);
  for (int i = 0; i + 1 < rank; ++i) r += (i ? ", d" : "d") + std::to_string(i);
  return "affine_map<(" + d + ") -> (" + r + ")>";
}
std::string iterators(int rank, bool lastIsReduction) {
  std::string s = "[";
  for (int i = 0; i < rank; ++i) {
    if (i) s += ", ";
    s += (lastIsReduction && i == rank - 1) ? "\"reduction\"" : "\"parallel\"";
  }
  return s + "]";
}

// The four generics a softmax over the last dimension decomposes into; defines `result`.
std::string decomposedSoftmax(const std::string &input, const std::string &result, const std::vector<int64_t> &dims,
                              const std::string &elem, const std::string &indent) {
  const int rank = static_cast<int>(dims.size());
  std::vector<int64_t> rdims(dims.begin(), dims.end() - 1);
  const std::string full = typeStr(dims, elem), red = typeStr(rdims, elem);
  const std::string id = identityMap(rank), dl = dropLastMap(rank);
  const std::string negInf = elem == "f16" ? "-6.550400e+04" : "-3.4028235e+38";
  std::ostringstream o;
  const std::string &in = indent;
  o << in << "%wtc_sm_neg_inf = arith.constant " << negInf << " : " << elem << "\n"
    << in << "%wtc_sm_zero = arith.constant 0.0 : " << elem << "\n"
    << in << "%wtc_sm_max0 = tensor.empty() : " << red << "\n"
    << in << "%wtc_sm_max_init = linalg.fill ins(%wtc_sm_neg_inf : " << elem << ") outs(%wtc_sm_max0 : " << red << ") -> " << red << "\n"
    << in << "%wtc_sm_max = linalg.generic {indexing_maps = [" << id << ", " << dl << "], iterator_types = " << iterators(rank, true) << "}\n"
    << in << "    ins(" << input << " : " << full << ") outs(%wtc_sm_max_init : " << red << ") {\n"
    << in << "  ^bb0(%in: " << elem << ", %acc: " << elem << "):\n"
    << in << "    %m = arith.maximumf %in, %acc : " << elem << "\n"
    << in << "    linalg.yield %m : " << elem << "\n"
    << in << "  } -> " << red << "\n"
    << in << "%wtc_sm_exp0 = tensor.empty() : " << full << "\n"
    << in << "%wtc_sm_exp = linalg.generic {indexing_maps = [" << id << ", " << dl << ", " << id << "], iterator_types = " << iterators(rank, false) << "}\n"
    << in << "    ins(" << input << ", %wtc_sm_max : " << full << ", " << red << ") outs(%wtc_sm_exp0 : " << full << ") {\n"
    << in << "  ^bb0(%x: " << elem << ", %m: " << elem << ", %out: " << elem << "):\n"
    << in << "    %d = arith.subf %x, %m : " << elem << "\n"
    << in << "    %e = math.exp %d : " << elem << "\n"
    << in << "    linalg.yield %e : " << elem << "\n"
    << in << "  } -> " << full << "\n"
    << in << "%wtc_sm_sum0 = tensor.empty() : " << red << "\n"
    << in << "%wtc_sm_sum_init = linalg.fill ins(%wtc_sm_zero : " << elem << ") outs(%wtc_sm_sum0 : " << red << ") -> " << red << "\n"
    << in << "%wtc_sm_sum = linalg.generic {indexing_maps = [" << id << ", " << dl << "], iterator_types = " << iterators(rank, true) << "}\n"
    << in << "    ins(%wtc_sm_exp : " << full << ") outs(%wtc_sm_sum_init : " << red << ") {\n"
    << in << "  ^bb0(%in: " << elem << ", %acc: " << elem << "):\n"
    << in << "    %s = arith.addf %in, %acc : " << elem << "\n"
    << in << "    linalg.yield %s : " << elem << "\n"
    << in << "  } -> " << red << "\n"
    << in << "%wtc_sm_div0 = tensor.empty() : " << full << "\n"
    << in << result << " = linalg.generic {indexing_maps = [" << id << ", " << dl << ", " << id << "], iterator_types = " << iterators(rank, false) << "}\n"
    << in << "    ins(%wtc_sm_exp, %wtc_sm_sum : " << full << ", " << red << ") outs(%wtc_sm_div0 : " << full << ") {\n"
    << in << "  ^bb0(%e: " << elem << ", %s: " << elem << ", %out: " << elem << "):\n"
    << in << "    %q = arith.divf %e, %s : " << elem << "\n"
    << in << "    linalg.yield %q : " << elem << "\n"
    << in << "  } -> " << full << "\n";
  return o.str();
}

} // namespace

bool parseChain(const std::string &rawText, ChainSpec &spec, std::string &diag) {
  const std::string text = expandAliases(stripComments(rawText));
  spec = ChainSpec();

  // ---- function signature
  static const std::regex fnRe(R"(func\.func\s+@([A-Za-z_][\w]*)\s*\()");
  std::smatch fm;
  if (!std::regex_search(text, fm, fnRe)) { diag = "no func.func found"; return false; }
  spec.funcName = fm[1].str();
  const size_t open = static_cast<size_t>(fm.position(0) + fm.length(0) - 1);
  const std::string args = parenGroup(text, open);
  const std::vector<TensorType> argTypes = allTensorTypes(args);
  if (argTypes.size() != 2) { diag = "expected exactly two tensor arguments (A, B), found " + std::to_string(argTypes.size()); return false; }
  const size_t arrow = text.find("->", open + args.size());
  TensorType resType;
  if (arrow == std::string::npos || !parseTensorType(text.substr(arrow, 200), resType)) { diag = "function result must be a static f16/f32 tensor"; return false; }

  // ---- the contraction
  size_t mm = text.find("linalg.batch_matmul");
  spec.batched = mm != std::string::npos;
  if (!spec.batched) mm = text.find("linalg.matmul");
  if (mm == std::string::npos) { diag = "no linalg.matmul / linalg.batch_matmul in the chain"; return false; }
  const size_t insPos = text.find("ins(", mm), outsPos = text.find("outs(", mm);
  if (insPos == std::string::npos || outsPos == std::string::npos || insPos - mm > 400 || outsPos - mm > 800) { diag = "matmul without ins(...) outs(...)"; return false; }
  const std::vector<TensorType> ins = allTensorTypes(parenGroup(text, insPos + 3));
  const std::vector<TensorType> outs = allTensorTypes(parenGroup(text, outsPos + 4));
  if (ins.size() != 2 || outs.size() != 1) { diag = "matmul needs two inputs and one output tensor"; return false; }
  const TensorType &a = ins[0], &b = ins[1], &c = outs[0];
  const size_t rank = spec.batched ? 3 : 2;
  if (a.dims.size() != rank || c.dims.size() != rank || (b.dims.size() != rank)) { diag = "matmul operand ranks do not match the op"; return false; }
  const size_t o = spec.batched ? 1 : 0;
  spec.batch = spec.batched ? a.dims[0] : 1;
  spec.bBatched = spec.batched;
  spec.M = a.dims[o]; spec.K = a.dims[o + 1]; spec.N = b.dims[o + 1];
  if (b.dims[o] != spec.K) { diag = "K mismatch between A and B"; return false; }
  if (c.dims[o] != spec.M || c.dims[o + 1] != spec.N || (spec.batched && (b.dims[0] != spec.batch || c.dims[0] != spec.batch))) { diag = "matmul result shape does not match its operands"; return false; }
  if (a.elem != b.elem) { diag = "A and B must share an element type"; return false; }
  if (a.dims != argTypes[0].dims || b.dims != argTypes[1].dims) { diag = "matmul must consume the function arguments (shapes differ)"; return false; }
  if (argTypes[0].elem != argTypes[1].elem) { diag = "A and B arguments must share an element type"; return false; }
  if (a.elem != argTypes[0].elem) {
    // the one accepted indirection: f32 arguments rounded to f16 by arith.truncf generics ahead of the matmul
    static const std::regex truncRe(R"(arith\.truncf\s+%[\w.]+\s*:\s*f32\s+to\s+f16)");
    const std::string head = text.substr(0, mm);
    const auto nTrunc = std::distance(std::sregex_iterator(head.begin(), head.end(), truncRe), std::sregex_iterator());
    if (!(argTypes[0].elem == "f32" && a.elem == "f16" && nTrunc >= 2)) {
      diag = "matmul must consume the function arguments directly, or f32 arguments rounded to f16 by arith.truncf";
      return false;
    }
  }
  spec.argType = argTypes[0].elem;
  spec.inType = a.elem;
  spec.accType = c.elem;
  if (resType.dims != c.dims) { diag = "function result shape must equal the matmul result shape"; return false; }
  spec.outType = resType.elem;

  // ---- the softmax
  spec.matmulCount = countContains(text, "linalg.matmul") + countContains(text, "linalg.batch_matmul");
  spec.genericCount = countContains(text, "linalg.generic");
  spec.reductionCount = countContains(text, "\"reduction\"");
  spec.expCount = countContains(text, "math.exp");
  spec.divCount = countContains(text, "arith.divf");
  if (spec.matmulCount != 1) { diag = "expected exactly one matmul in the chain"; return false; }
  static const std::regex smRe(R"(linalg\.softmax\s+dimension\(\s*([0-9]+)\s*\))");
  std::smatch sm;
  if (std::regex_search(text, sm, smRe)) {
    spec.namedSoftmax = true;
    if (std::stoul(sm[1].str()) != rank - 1) { diag = "linalg.softmax must reduce the last dimension (row softmax)"; return false; }
  } else {
    const bool hasMax = text.find("arith.maximumf") != std::string::npos || text.find("arith.maxnumf") != std::string::npos ||
                        text.find("arith.maxf") != std::string::npos;
    if (!hasMax || spec.expCount < 1 || spec.divCount < 1 || text.find("arith.addf") == std::string::npos || spec.reductionCount < 2) {
      diag = "no softmax found: need linalg.softmax, or max/exp/sum/div generics with two row reductions";
      return false;
    }
  }

  // ---- scale: constant factors applied with arith.mulf
  std::map<std::string, double> consts;
  static const std::regex cRe(R"((%[\w.]+)\s*=\s*arith\.constant\s+([-+0-9.eE]+(?:[eE][-+]?[0-9]+)?)\s*:\s*(?:f16|f32))");
  for (auto it = std::sregex_iterator(text.begin(), text.end(), cRe); it != std::sregex_iterator(); ++it)
    consts[(*it)[1].str()] = std::strtod((*it)[2].str().c_str(), nullptr);
  static const std::regex mulRe(R"(arith\.mulf\s+(%[\w.]+)\s*,\s*(%[\w.]+))");
  for (auto it = std::sregex_iterator(text.begin(), text.end(), mulRe); it != std::sregex_iterator(); ++it) {
    auto c1 = consts.find((*it)[1].str()), c2 = consts.find((*it)[2].str());
    if (c1 != consts.end()) spec.scale *= c1->second;
    else if (c2 != consts.end()) spec.scale *= c2->second;
    else { diag = "arith.mulf in the chain must have a constant operand (the scale)"; return false; }
  }
  diag.clear();
  return true;
}

bool parseChainFile(const std::string &path, ChainSpec &spec, std::string &diag) {
  const std::string text = readAll(path);
  if (text.empty()) { diag = "failed to read input MLIR: " + path; return false; }
  return parseChain(text, spec, diag);
}

std::string chainToJson(const ChainSpec &s) {
  char scale[64];
  snprintf(scale, sizeof scale, "%.9g", s.scale);
  std::ostringstream o;
  o << "{\n"
    << "  \"func\": \"" << s.funcName << "\",\n"
    << "  \"batch\": " << s.batch << ", \"M\": " << s.M << ", \"N\": " << s.N << ", \"K\": " << s.K << ",\n"
    << "  \"batched\": " << (s.batched ? "true" : "false") << ", \"b_batched\": " << (s.bBatched ? "true" : "false") << ",\n"
    << "  \"arg_dtype\": \"" << s.argType << "\", \"in_dtype\": \"" << s.inType << "\", \"acc_dtype\": \"" << s.accType << "\", \"out_dtype\": \"" << s.outType << "\",\n"
    << "  \"scale\": " << scale << ",\n"
    << "  \"softmax_form\": \"" << (s.namedSoftmax ? "named" : "decomposed") << "\"\n"
    << "}\n";
  return o.str();
}

bool canonicalizeMatmulSoftmaxChain(const std::string &inputPath, const std::string &outputPath, std::string &diagnostic) {
  trace::Span span("canonicalize");
  auto failWith = [&](const std::string &m) { diagnostic = m; span.fail(); return false; };
  if (inputPath.empty()) return failWith("input path is empty");
  if (outputPath.empty()) return failWith("output path is empty");
  if (!std::filesystem::exists(inputPath)) return failWith("input file not found: " + inputPath);
  const std::string input = readAll(inputPath);
  if (input.empty()) return failWith("failed to read input MLIR: " + inputPath);
  const std::filesystem::path dir = std::filesystem::path(outputPath).parent_path();
  const std::string logPath = (dir / "01.canonicalize.log").string();
  std::ostringstream log;
  log << "[wtc.canonicalize] input=" << inputPath << "\n";

  ChainSpec spec;
  std::string perr;
  if (!parseChain(input, spec, perr)) {
    log << "error: " << perr << "\n";
    writeAll(logPath, log.str());
    return failWith("chain recogniser rejected the input: " + perr + ", see " + logPath);
  }

  std::string text = expandAliases(input);   // the canonical form spells every type and map out
  if (spec.namedSoftmax) {
    // locate the statement  <result> = linalg.softmax dimension(d) ins(<x> : T) outs(... ) -> T
    static const std::regex stRe(R"((%[\w.]+)\s*=\s*linalg\.softmax\s+dimension\(\s*[0-9]+\s*\)\s*ins\(\s*(%[\w.]+)\s*:\s*(tensor<[^>]+>)\s*\))");
    std::smatch m;
    if (!std::regex_search(text, m, stRe)) { writeAll(logPath, log.str()); return failWith("cannot locate the linalg.softmax statement"); }
    const size_t start = static_cast<size_t>(m.position(0));
    size_t end = text.find("->", start + m.length(0));
    TensorType t;
    if (end == std::string::npos || !parseTensorType(m[3].str(), t)) { writeAll(logPath, log.str()); return failWith("malformed linalg.softmax statement"); }
    end = text.find('>', end + 2);   // end of the result tensor type
    size_t lineStart = text.rfind('\n', start);
    lineStart = lineStart == std::string::npos ? 0 : lineStart + 1;
    const std::string indent = text.substr(lineStart, start - lineStart);
    const std::string repl = decomposedSoftmax(m[2].str(), m[1].str(), t.dims, t.elem,
                                               indent.find_first_not_of(" \t") == std::string::npos ? indent : "    ");
    text = text.substr(0, lineStart) + repl + text.substr(end + 1);
    log << "[wtc.canonicalize] decomposed linalg.softmax over " << m[3].str() << " into max/exp/sum/div generics\n";
  }

  // like the output of an MLIR printer, the canonical form carries no comments
  {
    std::istringstream in(stripComments(text));
    std::ostringstream clean;
    std::string line;
    while (std::getline(in, line)) {
      const size_t last = line.find_last_not_of(" \t");
      if (last == std::string::npos) continue;
      clean << line.substr(0, last + 1) << '\n';
    }
    text = clean.str();
  }
  if (!writeAll(outputPath, text)) return failWith("failed to write canonicalized MLIR: " + outputPath);
  writeAll((dir / "chain.json").string(), chainToJson(spec));

  // acceptance checks on what was written
  const std::string body = stripComments(text);
  if (body.find("linalg.matmul") == std::string::npos && body.find("linalg.batch_matmul") == std::string::npos) { writeAll(logPath, log.str()); return failWith("canonicalized IR lost linalg.matmul unexpectedly"); }
  if (body.find("linalg.softmax") != std::string::npos) { writeAll(logPath, log.str()); return failWith("softmax decomposition did not run: linalg.softmax remains"); }
  if (body.find("math.exp") == std::string::npos || body.find("arith.divf") == std::string::npos) { writeAll(logPath, log.str()); return failWith("canonicalized IR does not contain expected softmax decomposition ops"); }
  ChainSpec again;
  if (!parseChain(text, again, perr) || again.M != spec.M || again.N != spec.N || again.K != spec.K || again.namedSoftmax) { writeAll(logPath, log.str()); return failWith("canonicalized IR does not parse back to the same chain: " + perr); }
  log << "[wtc.canonicalize] chain: batch=" << spec.batch << " M=" << spec.M << " N=" << spec.N << " K=" << spec.K << " in=" << spec.inType
      << " acc=" << spec.accType << " out=" << spec.outType << " scale=" << spec.scale << "\n[wtc.canonicalize] ok\n";
  writeAll(logPath, log.str());
  diagnostic.clear();
  return true;
}

bool tagTypicalChainOps(const std::string &inputPath, const std::string &outputPath, const std::string &tagsJsonPath,
                        std::string &diagnostic) {
  trace::Span span("tagging");
  auto failWith = [&](const std::string &m) { diagnostic = m; span.fail(); return false; };
  if (inputPath.empty()) return failWith("input path is empty");
  if (outputPath.empty()) return failWith("output path is empty");
  if (tagsJsonPath.empty()) return failWith("tags json path is empty");
  const std::string text = readAll(inputPath);
  if (text.empty()) return failWith("failed to read input MLIR for tagging: " + inputPath);

  const int matmul = countContains(text, "linalg.matmul") + countContains(text, "linalg.batch_matmul");
  const int generic = countContains(text, "linalg.generic");
  const int reduction = countContains(text, "\"reduction\"");
  const int exps = countContains(text, "math.exp");
  const int divs = countContains(text, "arith.divf");
  if (matmul == 0 || generic == 0) return failWith("tagging expects matmul + generic softmax decomposition in input");

  struct Tag { const char *needle, *alt, *name; bool done; };
  Tag tags[] = {{"linalg.matmul", "linalg.batch_matmul", "welder.matmul_anchor", false},
                {"\"reduction\"", nullptr, "welder.row_reduction", false},
                {"math.exp", nullptr, "welder.elementwise_exp", false},
                {"arith.divf", nullptr, "welder.elementwise_div", false}};
  std::ostringstream tagged;
  tagged << "// [wtc tagging] tags are emitted as comments for readability\n";
  std::istringstream in(text);
  std::string line;
  while (std::getline(in, line)) {
    const size_t cpos = line.find("//");
    const std::string code = cpos == std::string::npos ? line : line.substr(0, cpos);
    for (Tag &t : tags) {
      if (t.done) continue;
      if (code.find(t.needle) != std::string::npos || (t.alt && code.find(t.alt) != std::string::npos)) {
        tagged << "// wtc.tag: " << t.name << "\n";
        t.done = true;
      }
    }
    tagged << line << '\n';
  }
  if (!writeAll(outputPath, tagged.str())) return failWith("failed to write tagged MLIR: " + outputPath);

  std::ostringstream js;
  js << "{\n  \"pipeline\": \"typical_chain\",\n  \"source\": \"" << inputPath << "\",\n  \"counts\": {\n"
     << "    \"matmul\": " << matmul << ",\n    \"generic\": " << generic << ",\n    \"reduction_hints\": " << reduction << ",\n"
     << "    \"exp\": " << exps << ",\n    \"div\": " << divs << "\n  },\n  \"tags\": [\n"
     << "    \"welder.matmul_anchor\",\n    \"welder.row_reduction\",\n    \"welder.elementwise_exp\",\n    \"welder.elementwise_div\"\n  ]\n}\n";
  if (!writeAll(tagsJsonPath, js.str())) return failWith("failed to write tags json: " + tagsJsonPath);
  diagnostic.clear();
  return true;
}

} // namespace ir
} // namespace wtc
