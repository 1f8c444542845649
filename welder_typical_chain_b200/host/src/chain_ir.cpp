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
  return matchChain(text, spec, diag);
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
    << "  \"kind\": \"" << s.kind << "\",\n"
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
