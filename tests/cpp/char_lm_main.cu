// TEST INFRASTRUCTURE.  Minimal driver of dlcuda::run_char_lm (the reference's
// char-LM example, src/examples_api.cu) for the parity tests:
//   char_lm_main <epochs> <seq_len> <print_every> <gen_len> <weights path> [load]
//   char_lm_main xor <epochs> <print_every>          (dlcuda::run_xor, the reference's other example)
// Everything else keeps the defaults of dlcuda::CharLMConfig / dlcuda::XorConfig.  The program is
// linked once against the reference's layer headers and once against the
// headers of this repository; both runs must print the same training log.
#include <cstdlib>
#include <string>

#include <dl_cuda/examples.hpp>

int main(int argc, char **argv) {
  if (argc == 4 && std::string(argv[1]) == "xor") {
    dlcuda::XorConfig xor_cfg;
    xor_cfg.epochs = std::atoi(argv[2]);
    xor_cfg.print_every = std::atoi(argv[3]);
    return dlcuda::run_xor(xor_cfg);
  }
  if (argc < 6) return 2;
  dlcuda::CharLMConfig cfg;
  cfg.epochs = std::atoi(argv[1]);
  cfg.seq_len = std::atoi(argv[2]);
  cfg.print_every = std::atoi(argv[3]);
  cfg.gen_len = std::atoi(argv[4]);
  cfg.weights_path = argv[5];
  cfg.load_weights = argc > 6 && std::string(argv[6]) == "load";
  return dlcuda::run_char_lm(cfg);
}
