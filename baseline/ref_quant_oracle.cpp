// Oracle over the UNMODIFIED reference sources for the scalar codebooks' wire form and the whole-tensor codebook
// checkpoint of DenseModel::save_quantized (src/codebook.cpp, src/model.cpp:210-318). Test support only.
//
//   ref_quant_oracle codebook <data.f32> <n> <out.bin>     trains CodebookOIL8 and CodebookOIL4 on the n floats and writes
//                                                          [OIL8 blob][n index bytes][OIL4 blob][n index bytes]
//   ref_quant_oracle model <dir>                           writes <dir>/fp32.oil, <dir>/oil8.oil, <dir>/oil4.oil of one tiny DenseModel
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "oil/codebook.h"
#include "oil/model.h"

int main(int argc, char** argv) {
  if (argc >= 5 && std::strcmp(argv[1], "codebook") == 0) {
    const size_t n = (size_t)std::atoll(argv[3]);
    std::vector<float> x(n);
    std::ifstream f(argv[2], std::ios::binary);
    f.read((char*)x.data(), (std::streamsize)(n * 4));
    if (!f) return 3;
    std::ofstream o(argv[4], std::ios::binary);
    oil::CodebookOIL8 c8;
    c8.train(x.data(), n);
    std::vector<uint8_t> blob(c8.serialized_size());
    c8.serialize(blob.data());
    o.write((const char*)blob.data(), (std::streamsize)blob.size());
    for (size_t i = 0; i < n; ++i) { uint8_t q = c8.quantize(x[i]); o.write((const char*)&q, 1); }
    oil::CodebookOIL4 c4;
    c4.train(x.data(), n);
    blob.resize(c4.serialized_size());
    c4.serialize(blob.data());
    o.write((const char*)blob.data(), (std::streamsize)blob.size());
    for (size_t i = 0; i < n; ++i) { uint8_t q = c4.quantize(x[i]); o.write((const char*)&q, 1); }
    return 0;
  }
  if (argc >= 3 && std::strcmp(argv[1], "model") == 0) {
    oil::TransformerConfig cfg;
    cfg.vocab_size = 64; cfg.hidden_size = 32; cfg.num_layers = 1; cfg.num_heads = 2; cfg.head_dim = 16; cfg.ffn_hidden_size = 64;
    cfg.max_seq_len = 16;
    oil::DenseModel m(cfg);
    const std::string d = argv[2];
    m.save(d + "/fp32.oil");
    m.save_quantized(d + "/oil8.oil", oil::Format::OIL8);
    m.save_quantized(d + "/oil4.oil", oil::Format::OIL4);
    return 0;
  }
  std::fprintf(stderr, "usage: see the header of ref_quant_oracle.cpp\n");
  return 2;
}
