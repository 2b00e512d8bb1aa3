// Host-only driver for an AddressSanitizer + UndefinedBehaviorSanitizer build of the .param/.bin
// loader (the part of the runtime that parses untrusted files and needs no GPU).  For every
// `<stem>.param` named on the command line it loads the pair as it is, then again with the .bin cut
// at a spread of lengths and with single bytes of the .param overwritten: the loader must either
// succeed or fail with a message, never touch memory it does not own.  The reference runs its whole
// test suite under the same two sanitizers (.github/workflows/ci.yml:49-62) and feeds its loader the
// malformed graphs of test/Unit/malformed_graph_test.cpp.
#include <cstdio>
#include <fstream>
#include <iterator>
#include <string>
#include <vector>

#include "../../ncnn-compiler_b200/csrc/loader.h"

static std::vector<char> slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  return std::vector<char>(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
}

static void spill(const std::string& path, const std::vector<char>& bytes, size_t count) {
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  f.write(bytes.data(), static_cast<std::streamsize>(count));
}

static int load(const std::string& param, const std::string& bin) {
  nb::ModelDef model;
  std::string error;
  if (nb::load_model(param, bin, &model, &error)) {
    (void)nb::describe_model(model).size();
    return 1;
  }
  return error.empty() ? -1 : 0;  // a failure without a message is a defect
}

int main(int argc, char** argv) {
  if (argc < 3) {
    std::fprintf(stderr, "usage: %s <scratch-dir> <model.param>...\n", argv[0]);
    return 2;
  }
  const std::string scratch = argv[1];
  int loaded = 0, refused = 0, silent = 0, variants = 0;
  for (int a = 2; a < argc; ++a) {
    const std::string param = argv[a];
    const std::string bin = param.substr(0, param.size() - 6) + ".bin";
    const int whole = load(param, bin);
    (whole > 0 ? loaded : refused) += 1;
    if (whole < 0) ++silent;
    const std::vector<char> p = slurp(param), b = slurp(bin);
    const std::string tp = scratch + "/variant.param", tb = scratch + "/variant.bin";
    // the .bin cut short (and one byte long): must be refused or, at full length, accepted
    for (size_t cut : {size_t(0), size_t(1), size_t(3), b.size() / 3, b.size() / 2, b.size() > 0 ? b.size() - 1 : 0}) {
      if (cut > b.size()) continue;
      spill(tp, p, p.size());
      spill(tb, b, cut);
      if (load(tp, tb) < 0) ++silent;
      ++variants;
    }
    // single bytes of the .param replaced: digits, separators and letters in turn
    const char junk[] = {'0', '9', '-', ' ', '=', ',', 'x', '\n'};
    for (size_t i = 0, k = 0; i < p.size(); i += (p.size() / 97 + 1), ++k) {
      std::vector<char> q = p;
      q[i] = junk[k % sizeof(junk)];
      spill(tp, q, q.size());
      spill(tb, b, b.size());
      if (load(tp, tb) < 0) ++silent;
      ++variants;
    }
  }
  std::printf("files %d: loaded %d, refused %d; variants %d; failures without a message %d\n", argc - 2, loaded, refused,
              variants, silent);
  return silent == 0 ? 0 : 1;
}
