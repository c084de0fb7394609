// LoopSplit over printed Triton IR (include/triton_ext_loop_split_text.h). Line-oriented: the printer puts one
// operation on a line, a region's opening brace at the end of its operation's line and its closing brace on a line
// of its own, which is all the structure this rewrite needs.
#include "triton_ext_loop_split_text.h"

#include <cstdlib>
#include <cstring>
#include <map>
#include <set>
#include <string>
#include <vector>

namespace {

std::string trim(const std::string &s) {
  size_t a = s.find_first_not_of(" \t\r");
  if (a == std::string::npos) return "";
  size_t b = s.find_last_not_of(" \t\r");
  return s.substr(a, b - a + 1);
}

bool ends_with(const std::string &s, const char *suffix) {
  const size_t n = strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

// An SSA value name at s[pos]: %[A-Za-z0-9_.$-]+ with an optional #N result index. Advances pos.
bool parse_value(const std::string &s, size_t &pos, std::string &out) {
  if (pos >= s.size() || s[pos] != '%') return false;
  size_t p = pos + 1;
  while (p < s.size() && (isalnum(static_cast<unsigned char>(s[p])) || s[p] == '_' || s[p] == '.' || s[p] == '$' || s[p] == '-')) ++p;
  if (p == pos + 1) return false;
  if (p < s.size() && s[p] == '#') {
    size_t q = p + 1;
    while (q < s.size() && isdigit(static_cast<unsigned char>(s[q]))) ++q;
    if (q > p + 1) p = q;
  }
  out = s.substr(pos, p - pos);
  pos = p;
  return true;
}

bool eat(const std::string &s, size_t &pos, const char *lit) {
  const size_t n = strlen(lit);
  if (s.compare(pos, n, lit) != 0) return false;
  pos += n;
  return true;
}

// The text between the parenthesis at s[pos] and its partner. Advances pos past the partner.
bool parse_parens(const std::string &s, size_t &pos, std::string &inner) {
  if (pos >= s.size() || s[pos] != '(') return false;
  int depth = 0;
  for (size_t p = pos; p < s.size(); ++p) {
    if (s[p] == '(') ++depth;
    if (s[p] == ')' && --depth == 0) {
      inner = s.substr(pos + 1, p - pos - 1);
      pos = p + 1;
      return true;
    }
  }
  return false;
}

std::vector<std::string> split_list(const std::string &s) {
  std::vector<std::string> out;
  size_t a = 0;
  while (a <= s.size()) {
    size_t b = s.find(", ", a);
    if (b == std::string::npos) b = s.size();
    if (b > a) out.push_back(trim(s.substr(a, b - a)));
    a = b + 2;
  }
  return out;
}

struct ForHeader {
  std::string indent, results, iv, lo, hi, step, iters, types, ity;
  std::vector<std::pair<std::string, std::string>> iter_pairs;  // (region argument, initial value)
};

bool parse_for(const std::string &line, ForHeader &h) {
  const std::string t = trim(line);
  if (!ends_with(t, "{")) return false;
  const size_t at = line.find("scf.for ");
  if (at == std::string::npos) return false;
  const size_t first = line.find_first_not_of(" \t");
  h.indent = line.substr(0, first);
  h.results.clear();
  if (at > first) {
    const std::string lhs = line.substr(first, at - first);
    if (!ends_with(lhs, " = ") || lhs[0] != '%') return false;
    h.results = lhs.substr(0, lhs.size() - 3);
  }
  size_t p = at + 8;
  if (!parse_value(line, p, h.iv) || !eat(line, p, " = ") || !parse_value(line, p, h.lo) || !eat(line, p, " to ") ||
      !parse_value(line, p, h.hi) || !eat(line, p, " step ") || !parse_value(line, p, h.step))
    return false;
  h.iters.clear();
  h.types.clear();
  h.iter_pairs.clear();
  if (line.compare(p, 11, " iter_args(") == 0) {
    p += 10;
    if (!parse_parens(line, p, h.iters) || !eat(line, p, " -> ") || !parse_parens(line, p, h.types)) return false;
    for (const std::string &item : split_list(h.iters)) {
      const size_t eq = item.find(" = ");
      if (eq == std::string::npos) return false;
      h.iter_pairs.emplace_back(trim(item.substr(0, eq)), trim(item.substr(eq + 3)));
    }
  }
  const std::string tail = trim(line.substr(p));
  h.ity.clear();
  if (tail == "{") return true;  // index-typed loop: left alone by the caller
  if (tail.size() > 4 && tail.compare(0, 2, ": ") == 0 && ends_with(tail, " {")) {
    h.ity = trim(tail.substr(2, tail.size() - 4));
    return !h.ity.empty() && h.ity[0] == 'i';
  }
  return false;
}

struct Cmp {
  std::string indent, result, pred, lhs, rhs;
};

bool parse_cmp(const std::string &line, Cmp &c) {
  const size_t first = line.find_first_not_of(" \t");
  if (first == std::string::npos) return false;
  c.indent = line.substr(0, first);
  size_t p = first;
  if (!parse_value(line, p, c.result) || !eat(line, p, " = arith.cmpi ")) return false;
  const size_t comma = line.find(", ", p);
  if (comma == std::string::npos) return false;
  c.pred = line.substr(p, comma - p);
  p = comma + 2;
  if (!parse_value(line, p, c.lhs) || !eat(line, p, ", ") || !parse_value(line, p, c.rhs) || !eat(line, p, " : i")) return false;
  for (size_t q = p; q < line.size(); ++q)
    if (!isdigit(static_cast<unsigned char>(line[q]))) return trim(line.substr(q)).empty();
  return true;
}

// `%x = arith.constant <integer> : iN`
bool parse_int_constant(const std::string &line, std::string &name, long long &value) {
  size_t p = line.find_first_not_of(" \t");
  if (p == std::string::npos || !parse_value(line, p, name) || !eat(line, p, " = arith.constant ")) return false;
  char *end = nullptr;
  value = strtoll(line.c_str() + p, &end, 10);
  if (end == line.c_str() + p) return false;
  return strncmp(end, " : i", 4) == 0;
}

// Names a block of lines defines: operation results, loop induction variables and region arguments.
std::set<std::string> defined_inside(const std::vector<std::string> &lines, size_t a, size_t b) {
  std::set<std::string> names;
  for (size_t i = a; i < b; ++i) {
    const std::string &l = lines[i];
    const size_t first = l.find_first_not_of(" \t");
    if (first != std::string::npos && l[first] == '%') {
      const size_t eq = l.find(" = ", first);
      if (eq != std::string::npos)
        for (std::string tok : split_list(l.substr(first, eq - first))) {
          const size_t colon = tok.find(':');
          names.insert(colon == std::string::npos ? tok : tok.substr(0, colon));
        }
    }
    ForHeader h;
    if (parse_for(l, h)) {
      names.insert(h.iv);
      for (const auto &pr : h.iter_pairs) names.insert(pr.first);
    }
  }
  return names;
}

// `%r = op.name <anything with %operands> : types` -> result, name, operands, text after the name.
struct OpLine {
  std::string indent, result, name, rest;
  std::vector<std::string> operands;
};

bool parse_op(const std::string &line, OpLine &o) {
  const size_t first = line.find_first_not_of(" \t");
  if (first == std::string::npos || line[first] != '%') return false;
  o.indent = line.substr(0, first);
  size_t p = first;
  if (!parse_value(line, p, o.result) || !eat(line, p, " = ")) return false;
  const size_t sp = line.find(' ', p);
  o.name = line.substr(p, sp == std::string::npos ? std::string::npos : sp - p);
  o.rest = sp == std::string::npos ? "" : line.substr(sp + 1);
  o.operands.clear();
  for (size_t q = 0; q < o.rest.size();) {
    std::string v;
    if (o.rest[q] == '%' && parse_value(o.rest, q, v)) o.operands.push_back(v);
    else ++q;
  }
  return !o.name.empty();
}

// A tensor compare of the loop body that is all-true while iv + extent <= bound: the K mask of a tt.dot operand,
//   cmpi slt, expand/broadcast(addi(splat(iv), make_range[0, extent))), expand/broadcast(splat(bound))
struct MaskCmp {
  size_t line;
  std::string indent, result, i1_type;
};

struct Defs {
  const std::vector<std::string> *lines;
  std::map<std::string, size_t> body, global;
  bool lookup(const std::string &name, OpLine &o) const {
    auto it = body.find(name);
    if (it == body.end()) {
      it = global.find(name);
      if (it == global.end()) return false;
    }
    return parse_op((*lines)[it->second], o);
  }
  // Follow shape-only operations back to the value they reshape.
  bool root(std::string name, OpLine &o) const {
    for (int hops = 0; hops < 8; ++hops) {
      if (!lookup(name, o)) return false;
      if ((o.name == "tt.expand_dims" || o.name == "tt.broadcast") && o.operands.size() == 1) name = o.operands[0];
      else return true;
    }
    return false;
  }
};

bool make_range_from_zero(const OpLine &o, long long &extent) {
  if (o.name != "tt.make_range") return false;
  const size_t e = o.rest.find("end = "), s = o.rest.find("start = ");
  if (e == std::string::npos || s == std::string::npos) return false;
  extent = strtoll(o.rest.c_str() + e + 6, nullptr, 10);
  return strtoll(o.rest.c_str() + s + 8, nullptr, 10) == 0 && extent > 0;
}

// Is `line` a K mask in the sense above? On success: the extent of the index range and the bound's SSA name.
bool match_mask_cmp(const std::string &line, const Defs &defs, const std::string &iv, const std::set<std::string> &inside,
                    const std::map<std::string, long long> &consts, MaskCmp &out, long long &extent, std::string &bound,
                    int &adjust, long long &iv_scale) {
  iv_scale = 0;  // 0: the index is iv + range; c > 0: the index is the range alone and the bound is `bound - iv * c`
  OpLine c;
  if (!parse_op(line, c) || c.name != "arith.cmpi" || c.operands.size() != 2) return false;
  const size_t comma = c.rest.find(',');
  const std::string pred = trim(c.rest.substr(0, comma));
  if (pred == "slt" || pred == "ult") adjust = 0;
  else if (pred == "sle" || pred == "ule") adjust = 1;
  else return false;
  const size_t colon = c.rest.rfind(" : ");
  if (colon == std::string::npos) return false;
  std::string ty = trim(c.rest.substr(colon + 3));
  if (ty.compare(0, 7, "tensor<") != 0) return false;
  const size_t x = ty.rfind("xi");
  if (x == std::string::npos) return false;
  out.i1_type = ty.substr(0, x) + "xi1>";
  OpLine lhs, rhs, part;
  if (!defs.root(c.operands[0], lhs) || !defs.root(c.operands[1], rhs)) return false;
  if (rhs.name != "tt.splat" || rhs.operands.size() != 1) return false;
  if (make_range_from_zero(lhs, extent)) {
    // Loops that count K blocks: `arange(E) < bound - iv * c`, all-true while iv * c + E <= bound.
    OpLine left, prod;
    if (!defs.lookup(rhs.operands[0], left) || left.name != "arith.subi" || left.operands.size() != 2) return false;
    if (left.operands[0] == iv || inside.count(left.operands[0])) return false;
    if (!defs.lookup(left.operands[1], prod) || prod.name != "arith.muli" || prod.operands.size() != 2) return false;
    const std::string &x = prod.operands[0], &y = prod.operands[1];
    const std::string &scale = x == iv ? y : x;
    if ((x != iv && y != iv) || scale == iv) return false;
    auto it = consts.find(scale);
    if (it == consts.end() || it->second <= 0) return false;
    iv_scale = it->second;
    bound = left.operands[0];
    out.indent = c.indent;
    out.result = c.result;
    return true;
  }
  if (lhs.name != "arith.addi" || lhs.operands.size() != 2) return false;
  if (rhs.operands[0] == iv || inside.count(rhs.operands[0])) return false;  // the bound must be loop-invariant
  bool has_iv = false, has_range = false;
  for (const std::string &opnd : lhs.operands) {
    if (!defs.root(opnd, part)) return false;
    if (part.name == "tt.splat" && part.operands.size() == 1 && part.operands[0] == iv) has_iv = true;
    else if (make_range_from_zero(part, extent)) has_range = true;
  }
  if (!has_iv || !has_range) return false;
  bound = rhs.operands[0];
  out.indent = c.indent;
  out.result = c.result;
  return true;
}

// Index of the line that closes the region opened by lines[start], or -1.
long region_end(const std::vector<std::string> &lines, size_t start) {
  int depth = 0;
  for (size_t i = start; i < lines.size(); ++i) {
    const std::string t = trim(lines[i]);
    // "} else {" of scf.if and "} do {" of scf.while close one region and open the next: depth-neutral
    if (!t.empty() && t[0] == '}' && ends_with(t, "{")) continue;
    if (ends_with(t, "{")) {
      ++depth;
    } else if (!t.empty() && t[0] == '}') {
      if (--depth == 0) return static_cast<long>(i);
    }
  }
  return -1;
}

}  // namespace

namespace {

struct PredInfo {
  bool holds_below;  // the compare is true for iv < T (slt, sle) rather than for iv >= T (sge, sgt)
  int adjust;        // T = comparand + adjust
  bool equal;        // sge / sle (LoopSplit.cpp:35-44: CmpType::equal)
};

bool pred_info(const std::string &p, PredInfo &out) {
  static const std::map<std::string, PredInfo> table = {
      {"slt", {true, 0, false}},  {"ult", {true, 0, false}},  {"sle", {true, 1, true}},  {"ule", {true, 1, true}},
      {"sge", {false, 0, true}},  {"uge", {false, 0, true}},  {"sgt", {false, 1, false}}, {"ugt", {false, 1, false}}};
  auto it = table.find(p);
  if (it == table.end()) return false;
  out = it->second;
  return true;
}

std::string swapped(const std::string &p) {  // a < b  <=>  b > a
  static const std::map<std::string, std::string> m = {{"slt", "sgt"}, {"sgt", "slt"}, {"sle", "sge"}, {"sge", "sle"},
                                                       {"ult", "ugt"}, {"ugt", "ult"}, {"ule", "uge"}, {"uge", "ule"}};
  auto it = m.find(p);
  return it == m.end() ? "" : it->second;
}

std::string inverted(const std::string &p) {  // arith::invertPredicate, which the reference applies instead
  static const std::map<std::string, std::string> m = {{"slt", "sge"}, {"sge", "slt"}, {"sle", "sgt"}, {"sgt", "sle"},
                                                       {"ult", "uge"}, {"uge", "ult"}, {"ule", "ugt"}, {"ugt", "ule"}};
  auto it = m.find(p);
  return it == m.end() ? "" : it->second;
}

int split_text(const std::string &text, int mode, std::string &result, int32_t &n_split) {
  std::vector<std::string> lines;
  for (size_t a = 0; a <= text.size();) {
    size_t b = text.find('\n', a);
    if (b == std::string::npos) b = text.size();
    lines.push_back(text.substr(a, b - a));
    a = b + 1;
  }
  // SSA names repeat from one tt.func to the next (%0, %c1_i32, %cst ...): constants and definitions are looked
  // up among the lines of the function that holds the loop only. Lines outside any function form scope 0.
  std::vector<long> scope_of(lines.size(), 0);
  {
    long scope = 0, next_scope = 0;
    for (size_t k = 0; k < lines.size(); ++k) {
      const std::string t = trim(lines[k]);
      if (t.rfind("tt.func", 0) == 0 || t.rfind("func.func", 0) == 0) scope = ++next_scope;
      scope_of[k] = scope;
    }
  }
  std::map<long, std::map<std::string, long long>> consts_by_scope;
  for (size_t k = 0; k < lines.size(); ++k) {
    std::string name;
    long long v;
    if (parse_int_constant(lines[k], name, v)) consts_by_scope[scope_of[k]][name] = v;
  }
  std::vector<std::string> out;
  n_split = 0;
  for (size_t i = 0; i < lines.size();) {
    ForHeader h;
    if (!parse_for(lines[i], h)) {
      out.push_back(lines[i++]);
      continue;
    }
    const long end = region_end(lines, i);
    if (end < 0) return 2;
    const size_t b0 = i + 1, b1 = static_cast<size_t>(end);
    const std::set<std::string> inside = defined_inside(lines, b0, b1);
    const long scope = scope_of[i];
    const std::map<std::string, long long> &consts = consts_by_scope[scope];
    const auto step_it = consts.find(h.step);
    long chosen = -1;
    Cmp cmp;
    std::string pred, comparand;
    PredInfo info{};
    if (!h.ity.empty() && step_it != consts.end() && step_it->second > 0) {
      for (size_t bi = b0; bi < b1; ++bi) {
        Cmp c;
        if (!parse_cmp(lines[bi], c)) continue;
        std::string p = c.pred, x = c.lhs, y = c.rhs;
        if (y == h.iv && x != h.iv) {
          p = mode == TXLS_AS_WRITTEN ? inverted(p) : swapped(p);
          std::swap(x, y);
        }
        PredInfo pi{};
        if (x != h.iv || y == h.iv || !pred_info(p, pi) || inside.count(y)) continue;
        if (mode == TXLS_INTENT && p[0] == 'u') {
          // An unsigned compare is monotone in the induction variable only while that is non-negative, and the
          // comparand is a run-time value that may have its sign bit set (then `ult` holds, and `uge` fails, for
          // every non-negative iv). With a constant lower bound >= 0 the split is made safe by a run-time guard
          // below; otherwise this compare is left alone.
          const auto lo_it = consts.find(h.lo);
          if (lo_it == consts.end() || lo_it->second < 0) continue;
        }
        chosen = static_cast<long>(bi);
        cmp = c;
        pred = p;
        comparand = y;
        info = pi;
        break;
      }
    }
    // No scalar compare of the induction variable: look for the K masks of the loads instead (the reference leaves
    // this open, LoopSplit.cpp:105 "TODO: add support for mask logic"). All masks over the same index range and
    // bound are all-true while iv + extent <= bound, so the loop splits there and its first half loses them.
    std::vector<MaskCmp> masks;
    long long mask_extent = 0, mask_scale = 0;
    std::string mask_bound;
    int mask_adjust = 0;
    if (chosen < 0 && mode == TXLS_INTENT && !h.ity.empty() && step_it != consts.end() && step_it->second > 0) {
      Defs defs;
      defs.lines = &lines;
      for (size_t k = 0; k < lines.size(); ++k) {
        OpLine o;
        if (parse_op(lines[k], o)) {
          if (scope_of[k] != scope) continue;
          defs.global.emplace(o.result, k);
          if (k >= b0 && k < b1) defs.body.emplace(o.result, k);
        }
      }
      for (size_t bi = b0; bi < b1; ++bi) {
        MaskCmp mc;
        long long e = 0;
        std::string bnd;
        int adj = 0;
        long long scale = 0;
        if (!match_mask_cmp(lines[bi], defs, h.iv, inside, consts, mc, e, bnd, adj, scale)) continue;
        if (masks.empty()) {
          mask_extent = e;
          mask_bound = bnd;
          mask_adjust = adj;
          mask_scale = scale;
        } else if (e != mask_extent || bnd != mask_bound || adj != mask_adjust || scale != mask_scale) {
          continue;  // another range or bound: stays a mask in both halves
        }
        mc.line = bi;
        masks.push_back(mc);
      }
    }
    if (chosen < 0 && masks.empty()) {  // not a loop to split; loops nested inside it are still looked at
      out.push_back(lines[i++]);
      continue;
    }
    const std::string tag = "%ls" + std::to_string(n_split);
    const std::string &in = h.indent, &ty = h.ity;
    const long long stepv = step_it->second;
    std::vector<std::string> pre;
    std::string midp;
    bool first_true;
    if (chosen < 0) {
      // iv + extent <= bound + adjust  <=>  iv < bound - (extent - 1 - adjust): the threshold of an `slt` compare.
      if (mask_scale == 0) {
        pre.push_back(in + tag + "_e = arith.constant " + std::to_string(mask_extent - 1 - mask_adjust) + " : " + ty);
        pre.push_back(in + tag + "_b = arith.subi " + mask_bound + ", " + tag + "_e : " + ty);
      } else {
        // iv * c + extent <= bound + adjust  <=>  iv < floor((bound + adjust - extent) / c) + 1
        pre.push_back(in + tag + "_e = arith.constant " + std::to_string(mask_extent - mask_adjust) + " : " + ty);
        pre.push_back(in + tag + "_s = arith.constant " + std::to_string(mask_scale) + " : " + ty);
        pre.push_back(in + tag + "_o = arith.constant 1 : " + ty);
        pre.push_back(in + tag + "_g = arith.subi " + mask_bound + ", " + tag + "_e : " + ty);
        pre.push_back(in + tag + "_f = arith.floordivsi " + tag + "_g, " + tag + "_s : " + ty);
        pre.push_back(in + tag + "_b = arith.addi " + tag + "_f, " + tag + "_o : " + ty);
      }
      comparand = tag + "_b";
      info = PredInfo{true, 0, false};
    }
    if (mode == TXLS_AS_WRITTEN) {
      const bool greater = !info.holds_below;
      midp = comparand;
      if (info.equal) {
        pre.push_back(in + tag + "_inc = arith.constant " + std::to_string(greater ? -stepv : stepv) + " : " + ty);
        pre.push_back(in + tag + "_t = arith.addi " + comparand + ", " + tag + "_inc : " + ty);
        midp = tag + "_t";
      }
      if (stepv != 1) {
        pre.push_back(in + tag + "_d = arith.subi " + midp + ", " + h.lo + " : " + ty);
        pre.push_back(in + tag + "_r = arith.remui " + tag + "_d, " + h.step + " : " + ty);
        pre.push_back(in + tag + "_u = arith.subi " + h.step + ", " + tag + "_r : " + ty);
        pre.push_back(in + tag + "_e = arith.addi " + tag + "_d, " + tag + "_u : " + ty);
        pre.push_back(in + tag + "_mid = arith.addi " + h.lo + ", " + tag + "_e : " + ty);
        midp = tag + "_mid";
      }
      first_true = !greater;
    } else {
      std::string thr = comparand;
      pre.push_back(in + tag + "_c0 = arith.constant 0 : " + ty);
      if (info.adjust) {
        pre.push_back(in + tag + "_c1 = arith.constant 1 : " + ty);
        pre.push_back(in + tag + "_t = arith.addi " + comparand + ", " + tag + "_c1 : " + ty);
        thr = tag + "_t";
      }
      pre.push_back(in + tag + "_d = arith.subi " + thr + ", " + h.lo + " : " + ty);
      pre.push_back(in + tag + "_p = arith.maxsi " + tag + "_d, " + tag + "_c0 : " + ty);
      pre.push_back(in + tag + "_q = arith.ceildivsi " + tag + "_p, " + h.step + " : " + ty);
      pre.push_back(in + tag + "_m = arith.muli " + tag + "_q, " + h.step + " : " + ty);
      pre.push_back(in + tag + "_a = arith.addi " + h.lo + ", " + tag + "_m : " + ty);
      pre.push_back(in + tag + "_h = arith.maxsi " + h.hi + ", " + h.lo + " : " + ty);
      if (chosen >= 0 && pred[0] == 'u') {
        // comparand with the sign bit set = an unsigned value above every non-negative iv: the compare has one
        // value over the whole range, which stays in the first copy (mid = hi)
        pre.push_back(in + tag + "_cl = arith.minsi " + tag + "_a, " + tag + "_h : " + ty);
        pre.push_back(in + tag + "_neg = arith.cmpi slt, " + comparand + ", " + tag + "_c0 : " + ty);
        pre.push_back(in + tag + "_mid = arith.select " + tag + "_neg, " + tag + "_h, " + tag + "_cl : " + ty);
      } else {
        pre.push_back(in + tag + "_mid = arith.minsi " + tag + "_a, " + tag + "_h : " + ty);
      }
      midp = tag + "_mid";
      first_true = info.holds_below;
    }
    const size_t n_res = h.iter_pairs.size();
    const std::string main_name = tag + "_main";
    std::string head1 = in, head2 = in;
    if (n_res) head1 += main_name + (n_res == 1 ? "" : ":" + std::to_string(n_res)) + " = ";
    if (!h.results.empty()) head2 += h.results + " = ";
    head1 += "scf.for " + h.iv + " = " + h.lo + " to " + midp + " step " + h.step;
    head2 += "scf.for " + h.iv + " = " + midp + " to " + h.hi + " step " + h.step;
    if (n_res) {
      std::string second;
      for (size_t k = 0; k < n_res; ++k) {
        if (k) second += ", ";
        second += h.iter_pairs[k].first + " = " + main_name + (n_res == 1 ? "" : "#" + std::to_string(k));
      }
      head1 += " iter_args(" + h.iters + ") -> (" + h.types + ")";
      head2 += " iter_args(" + second + ") -> (" + h.types + ")";
    }
    head1 += "  : " + ty + " {";
    head2 += "  : " + ty + " {";
    out.insert(out.end(), pre.begin(), pre.end());
    for (int copy = 0; copy < 2; ++copy) {
      out.push_back(copy == 0 ? head1 : head2);
      const bool value = (copy == 0) == first_true;
      for (size_t bi = b0; bi < b1; ++bi) {
        const MaskCmp *mask = nullptr;
        for (const MaskCmp &mc : masks)
          if (mc.line == bi) mask = &mc;
        if (static_cast<long>(bi) == chosen)
          out.push_back(cmp.indent + cmp.result + " = arith.constant " + (value ? "true" : "false"));
        else if (mask && copy == 0)
          out.push_back(mask->indent + mask->result + " = arith.constant dense<true> : " + mask->i1_type);
        else
          out.push_back(lines[bi]);
      }
      out.push_back(lines[b1]);
    }
    ++n_split;
    i = b1 + 1;
  }
  result.clear();
  for (size_t k = 0; k < out.size(); ++k) {
    result += out[k];
    if (k + 1 < out.size()) result += '\n';
  }
  if (result.empty() || result.back() != '\n') result += '\n';
  return 0;
}

}  // namespace

extern "C" {

int tx_loop_split_text(const char *ir_text, int mode, char **out_text, int32_t *loops_split) {
  if (!ir_text || !out_text || !loops_split || (mode != TXLS_INTENT && mode != TXLS_AS_WRITTEN)) return 1;
  std::string result;
  int32_t n = 0;
  const int rc = split_text(ir_text, mode, result, n);
  if (rc != 0) return rc;
  char *buf = static_cast<char *>(malloc(result.size() + 1));
  if (!buf) return 1;
  memcpy(buf, result.c_str(), result.size() + 1);
  *out_text = buf;
  *loops_split = n;
  return 0;
}

void tx_loop_split_free(char *text) { free(text); }

}  // extern "C"
