// Timing driver over the UNMODIFIED reference sources, through the reference's public API only:
// oil::DenseModel + oil::Trainer::compile/train_step + oil::AdamW (src/trainer_core.cpp:70-88,227-290,
// src/optimizer.cpp:91-119), the loop of bench/bench_training.cpp:75-130 plus the optimizer step, and for the
// tiny configuration also DenseModel::save and Generator::generate_tokens (src/generator.cpp:14-63).
// None of this framework's code is linked in. Token ids come from a file of int32 written by the caller
// (Zipf(1.1) ids, the same stream our own arm trains on).
//
//   ref_train_bench <ids.i32> <layers> <hidden> <heads> <ffn> <vocab> <seq> <batch> <warmup> <steps>
//                   <gelu 0|1> <lr> <wd> [<export.oil> <greedy_tokens>]
//
// Prints one JSON object: seconds per step (std::chrono, as every reference benchmark times), tokens/s, losses.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

#include "oil/generator.h"
#include "oil/model.h"
#include "oil/optimizer.h"
#include "oil/sampler.h"
#include "oil/tensor.h"
#include "oil/tokenizer.h"
#include "oil/trainer.h"

// A tokenizer that never ends a generation early: generate_tokens() reads eos_id() of the tokenizer it is given.
struct IdTokenizer : oil::Tokenizer {
  int v;
  explicit IdTokenizer(int vocab) : v(vocab) {}
  std::vector<int> encode(const std::string& t) override { return std::vector<int>(t.begin(), t.end()); }
  std::string decode(const std::vector<int>& ids) override { return std::string(ids.begin(), ids.end()); }
  int vocab_size() const override { return v; }
  int bos_id() const override { return -1; }
  int eos_id() const override { return -1; }
};

static double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, char** argv) {
  if (argc < 14) {
    std::fprintf(stderr, "usage: see the header of ref_train_bench.cpp\n");
    return 2;
  }
  const std::string ids_path = argv[1];
  const int64_t L = std::atoll(argv[2]), E = std::atoll(argv[3]), H = std::atoll(argv[4]), F = std::atoll(argv[5]);
  const int64_t V = std::atoll(argv[6]), S = std::atoll(argv[7]), B = std::atoll(argv[8]);
  const int warmup = std::atoi(argv[9]), steps = std::atoi(argv[10]);
  const bool gelu = std::atoi(argv[11]) != 0;
  const float lr = (float)std::atof(argv[12]), wd = (float)std::atof(argv[13]);
  const std::string export_path = argc > 14 ? argv[14] : "";
  const int greedy = argc > 15 ? std::atoi(argv[15]) : 0;

  std::ifstream f(ids_path, std::ios::binary);
  std::vector<int32_t> ids((size_t)(warmup + steps) * B * S + 1);
  f.read((char*)ids.data(), (std::streamsize)(ids.size() * 4));
  if (!f) {
    std::fprintf(stderr, "ids file too short\n");
    return 3;
  }

  oil::TransformerConfig cfg;
  cfg.vocab_size = V;
  cfg.hidden_size = E;
  cfg.num_layers = L;
  cfg.num_heads = H;
  cfg.head_dim = E / H;
  cfg.ffn_hidden_size = F;
  cfg.max_seq_len = S;
  cfg.activation = gelu ? oil::Activation::GELU : oil::Activation::SiLU;
  oil::DenseModel model(cfg);

  oil::Trainer trainer(&model, nullptr);
  oil::AdamW opt(lr, 0.9f, 0.999f, 1e-8f, wd);
  oil::TrainConfig tc;
  tc.learning_rate = lr;
  tc.weight_decay = wd;
  tc.batch_size = (int)B;
  tc.seq_length = (int)S;
  tc.schedule = oil::AdamW::Schedule::CONSTANT;
  trainer.compile(&opt, tc);

  oil::Tensor x({B, S}, oil::DType::F32), y({B * S}, oil::DType::F32);
  double t0 = 0, first = 0, last = 0;
  for (int it = 0; it < warmup + steps; ++it) {
    if (it == warmup) t0 = now_s();
    const int32_t* p = ids.data() + (size_t)it * B * S;
    float* xd = x.data<float>();
    float* yd = y.data<float>();
    for (int64_t i = 0; i < B * S; ++i) {
      xd[i] = (float)p[i];
      yd[i] = (float)p[i + 1];
    }
    const float loss = trainer.train_step(x, y);
    if (it == 0) first = loss;
    last = loss;
  }
  const double dt = (now_s() - t0) / (steps > 0 ? steps : 1);

  double decode_tps = 0;
  int n_dec = 0;
  if (!export_path.empty()) {
    model.save(export_path);
    if (greedy > 0) {
      oil::SamplerConfig sp;   // greedy: top-1 of the full distribution
      sp.temperature = 1.0f;
      sp.top_k = 1;
      sp.top_p = 1.0f;
      sp.max_tokens = greedy;
      IdTokenizer tok((int)V);
      oil::Generator gen(&model, &tok);
      std::vector<int> prompt(ids.begin(), ids.begin() + 16);
      const double d0 = now_s();
      std::vector<int> out = gen.generate_tokens(prompt, sp);
      const double d1 = now_s();
      n_dec = (int)out.size() - (int)prompt.size();
      decode_tps = n_dec / (d1 - d0);
    }
  }
  std::printf("{\"s_per_step\": %.6f, \"tokens_per_s\": %.4f, \"tokens_per_step\": %lld, \"loss_first\": %.5f, \"loss_last\": %.5f, "
              "\"params\": %lld, \"decode_tokens\": %d, \"decode_tokens_per_s\": %.3f}\n",
              dt, (double)(B * S) / dt, (long long)(B * S), first, last, (long long)model.param_count(), n_dec, decode_tps);
  return 0;
}
