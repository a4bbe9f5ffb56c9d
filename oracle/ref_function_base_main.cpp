// Driver around the REFERENCE's own ncu_function_base (scheduler/kernel_key.hpp:13-55), compiled from the
// reference tree where it lies (-I <reference>/scheduler).  Test infrastructure: reads one symbol per line on
// stdin, prints "symbol<TAB>short name".  Used to generate tests/golden/function_base.tsv.
#include <iostream>
#include <string>

#include "kernel_key.hpp"

int main() {
  std::string line;
  while (std::getline(std::cin, line)) std::cout << line << '\t' << ncu_function_base(line.c_str()) << '\n';
  return 0;
}
