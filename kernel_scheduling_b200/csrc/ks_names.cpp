// ks_names.cpp -- kernel symbol -> the short name the key dictionary is built on.
//
// Same result as the reference's ncu_function_base (scheduler/kernel_key.hpp:13-55): demangle, then keep only the
// function's own identifier -- no return type, namespaces, template arguments or parameter list.  Host-side work
// (strings, once per distinct symbol at ingest), so it lives outside the CUDA stages.
#include <cxxabi.h>

#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/ks_b200.h"

namespace {

std::string function_base(const char* symbol) {
  const std::string original = symbol ? symbol : "";
  std::string text = original;
  if (text.rfind("_Z", 0) == 0) {
    int status = -1;
    char* plain = abi::__cxa_demangle(symbol, nullptr, nullptr, &status);
    if (plain && status == 0) text = plain;
    std::free(plain);
  }
  // "(anonymous namespace)" would read as a parameter list below
  static const char kAnon[] = "(anonymous namespace)";
  for (size_t at = text.find(kAnon); at != std::string::npos; at = text.find(kAnon)) text.replace(at, sizeof(kAnon) - 1, "anonymous");

  // Walk to the '(' that opens the function's parameters.  Angle brackets nest only outside round / square / curly
  // brackets (inside those, '<' and '>' are comparison operators), so the nesting is a run of open angles followed
  // by a run of open "expression" brackets: two depths describe it, plus where each open angle sits.
  std::vector<size_t> open_angles;
  size_t expr_depth = 0;
  size_t cut = text.size();
  size_t closed_at = std::string::npos, closed_from = 0;  // the template argument list closed last: ['<' .. '>']
  for (size_t i = 0; i < text.size(); ++i) {
    const char ch = text[i];
    if (ch == '(' || ch == '[' || ch == '{') {
      if (ch == '(' && expr_depth == 0 && open_angles.empty()) { cut = i; break; }
      ++expr_depth;
    } else if (ch == ')' || ch == ']' || ch == '}') {
      if (expr_depth) --expr_depth;
      else if (!open_angles.empty()) open_angles.pop_back();
    } else if (ch == '<' && expr_depth == 0) {
      open_angles.push_back(i);
    } else if (ch == '>' && expr_depth == 0 && !open_angles.empty()) {
      closed_at = i;
      closed_from = open_angles.back();
      open_angles.pop_back();
    }
  }
  text.erase(cut);
  while (!text.empty() && text.back() == ' ') text.pop_back();
  if (!text.empty() && text.back() == '>' && closed_at == text.size() - 1) text.erase(closed_from);  // own template arguments

  const size_t blank = text.rfind(' ');  // return type
  if (blank != std::string::npos) text.erase(0, blank + 1);
  const size_t scope = text.rfind("::");  // namespaces and classes
  if (scope != std::string::npos) text.erase(0, scope + 2);
  return text.empty() ? original : text;
}

}  // namespace

extern "C" int64_t ks_function_base(const char* symbol, char* out, uint64_t capacity) {
  if (!out || capacity == 0) return -KS_ERR_ARG;
  const std::string s = function_base(symbol);
  if (s.size() + 1 > capacity) return -KS_ERR_CAPACITY;
  std::memcpy(out, s.c_str(), s.size() + 1);
  return (int64_t)s.size();
}
