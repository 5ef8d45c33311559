// Minimal stand-in for the few pieces of the {fmt} library that the reference's COMPILER sources
// use (fmt::print with "{}" placeholders in its logger, two fmt::formatter specialisations).  The
// reference pins {fmt} 9.1.0, which this image does not have (no network) and whose newer releases
// dropped the calls it uses.  TEST INFRASTRUCTURE: only the fixture generator of this directory builds
// the reference compiler against it, to produce compiled-program artefacts; nothing else includes it.
#pragma once
#include <cstdio>
#include <fstream>
#include <iostream>
#include <iterator>
#include <sstream>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <utility>

namespace fmt {

class format_parse_context {
 public:
  using iterator = const char*;
  constexpr format_parse_context(const char* b, const char* e) : b_(b), e_(e) {}
  constexpr iterator begin() const { return b_; }
  constexpr iterator end() const { return e_; }
  void on_error(const char* msg) const { throw std::runtime_error(msg); }

 private:
  const char *b_, *e_;
};

class format_context {
 public:
  using iterator = std::back_insert_iterator<std::string>;
  explicit format_context(std::string& s) : s_(s) {}
  iterator out() { return std::back_inserter(s_); }

 private:
  std::string& s_;
};

template <typename T, typename = void>
struct formatter;  // specialised by the user for their types

namespace detail {
template <typename T, typename = void>
struct has_formatter : std::false_type {};
template <typename T>
struct has_formatter<T, std::void_t<decltype(formatter<T>().format(std::declval<const T&>(), std::declval<format_context&>()))>>
    : std::true_type {};

template <typename T>
void append(std::string& out, const T& v) {
  if constexpr (has_formatter<T>::value) {
    format_context ctx(out);
    formatter<T>().format(v, ctx);
  } else if constexpr (std::is_same_v<T, unsigned char> || std::is_same_v<T, signed char>) {
    out += std::to_string((int)v);
  } else {
    std::ostringstream s;
    s << v;
    out += s.str();
  }
}
inline void vformat(std::string& out, const char* f) { out += f; }
template <typename A, typename... Rest>
void vformat(std::string& out, const char* f, const A& a, const Rest&... rest) {
  for (; *f; f++) {
    if (f[0] == '{' && f[1] == '}') {
      append(out, a);
      vformat(out, f + 2, rest...);
      return;
    }
    out += *f;
  }
}
}  // namespace detail

template <typename... Args>
std::string format(const char* f, const Args&... args) {
  std::string s;
  detail::vformat(s, f, args...);
  return s;
}
template <typename... Args>
std::string format(const std::string& f, const Args&... args) { return format(f.c_str(), args...); }

template <typename... Args>
void print(const char* f, const Args&... args) {
  const std::string s = format(f, args...);
  std::fwrite(s.data(), 1, s.size(), stdout);
}

template <typename Out, typename... Args>
Out format_to(Out out, const char* f, const Args&... args) {
  const std::string s = format(f, args...);
  for (char c : s) *out++ = c;
  return out;
}

}  // namespace fmt
