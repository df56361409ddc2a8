// Draws tokens with adarsh-sgh/edgelm's own Sampler (include/edgelm/tokenizer.hpp,
// src/tokenizer.cpp:191-211); built and run only by make_golden.py.
//   sampler_driver temperature top_k seed n_rows vocab < logits.f32   -> one token id a line
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "edgelm/tokenizer.hpp"

int main(int argc, char** argv) {
  if (argc != 6) return 2;
  const float temp = std::atof(argv[1]);
  const int k = std::atoi(argv[2]);
  const unsigned long long seed = std::strtoull(argv[3], nullptr, 10);
  const int n = std::atoi(argv[4]), vocab = std::atoi(argv[5]);
  edgelm::Sampler sampler({temp, k, seed});
  std::vector<float> row(vocab);
  for (int i = 0; i < n; ++i) {
    if (std::fread(row.data(), sizeof(float), vocab, stdin) != static_cast<size_t>(vocab)) return 1;
    std::printf("%d\n", sampler.sample(row.data(), vocab));
  }
  return 0;
}
