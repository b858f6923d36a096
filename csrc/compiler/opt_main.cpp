// nkipy-b200-opt: text-in / text-out driver of the native pass pipeline (the role of the
// reference's nkipy-opt binary, nkigen/mlir/tools/nkipy-opt/nkipy-opt.cpp:32-51).
//
//   nkipy-b200-opt [--pass NAME]... [--pipeline] [--stop-after X] [--dump-dir DIR] [--dump-start N]
//                  [--smem-capacity BYTES] [--tmem-columns N] [--sm-count N] [--fast-math]
//                  [--list-passes] [-o OUT] [INPUT | -]
//
// With --pass options the named passes run in the given order; otherwise (or with
// --pipeline) the default pipeline runs, optionally stopped after a pass / group / index.
// The resulting IR goes to stdout (or -o).  Errors go to stderr with exit code 1.
#include <fstream>
#include <iostream>
#include <sstream>

#include "passes.h"

int main(int argc, char** argv) {
  using namespace b200c;
  std::vector<std::string> passes;
  std::string stop_after, dump_dir, input = "-", output;
  bool pipeline = false;
  int dump_start = 1;
  PassOptions opts;
  try {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      auto next = [&](const char* what) -> std::string {
        if (i + 1 >= argc) throw CompileError(std::string("missing value for ") + what);
        return argv[++i];
      };
      if (a == "--pass") passes.push_back(next("--pass"));
      else if (a.rfind("--pass=", 0) == 0) passes.push_back(a.substr(7));
      else if (a == "--pipeline") pipeline = true;
      else if (a == "--stop-after") stop_after = next("--stop-after");
      else if (a == "--dump-dir") dump_dir = next("--dump-dir");
      else if (a == "--dump-start") dump_start = std::stoi(next("--dump-start"));
      else if (a == "--smem-capacity") opts.smem_capacity = std::stoll(next("--smem-capacity"));
      else if (a == "--tmem-columns") opts.tmem_columns = std::stoll(next("--tmem-columns"));
      else if (a == "--sm-count") opts.sm_count = std::stoi(next("--sm-count"));
      else if (a == "--target") opts.target = next("--target");
      else if (a == "--fast-math") opts.fast_math = true;
      else if (a == "-o") output = next("-o");
      else if (a == "--list-passes") {
        for (const PassInfo& p : default_pipeline()) std::cout << p.name << "\t" << p.group << "\t" << p.description << "\n";
        return 0;
      } else if (a == "-h" || a == "--help") {
        std::cout << "usage: nkipy-b200-opt [--pass NAME]... [--pipeline] [--stop-after X] [--dump-dir DIR] "
                     "[--smem-capacity N] [--fast-math] [--list-passes] [-o OUT] [INPUT|-]\n";
        return 0;
      } else if (a[0] == '-' && a != "-") throw CompileError("unknown option " + a);
      else input = a;
    }
    std::stringstream buf;
    if (input == "-") buf << std::cin.rdbuf();
    else {
      std::ifstream f(input);
      if (!f) throw CompileError("cannot open " + input);
      buf << f.rdbuf();
    }
    std::string result = (passes.empty() || pipeline) ? run_pipeline(buf.str(), stop_after, dump_dir, opts, dump_start)
                                                       : apply_passes(buf.str(), passes, opts);
    if (output.empty()) std::cout << result;
    else {
      std::ofstream f(output);
      f << result;
    }
  } catch (const std::exception& e) {
    std::cerr << "nkipy-b200-opt: error: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
