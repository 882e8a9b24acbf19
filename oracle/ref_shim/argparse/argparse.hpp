// No-op stand-in for p-ranav/argparse: parse_args() is compiled but never
// called by the oracle driver.
#ifndef ORACLE_SHIM_ARGPARSE_HPP
#define ORACLE_SHIM_ARGPARSE_HPP
#include <optional>
#include <ostream>
#include <stdexcept>
#include <string>
namespace argparse {
struct Argument {
  Argument &help(const char *) { return *this; }
  template <class T> Argument &default_value(T) { return *this; }
  template <class T> Argument &implicit_value(T) { return *this; }
  template <char C, class T> Argument &scan() { return *this; }
};
struct ArgumentParser {
  Argument arg_;
  explicit ArgumentParser(const char *) {}
  template <class... A> Argument &add_argument(A...) { return arg_; }
  void parse_args(int, const char **) {}
  bool is_used(const char *) const { return false; }
  template <class T = std::string> T get(const char *) const { return T(); }
  template <class T = std::string> std::optional<T> present(const char *) const { return std::nullopt; }
};
inline std::ostream &operator<<(std::ostream &os, const ArgumentParser *) { return os; }
} // namespace argparse
#endif
