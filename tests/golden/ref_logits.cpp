// Runs the reference project's own LFM3 model code on its CPU backend and writes last-token logits.
// Built and run by make_golden.py; links the reference's libraries, contains none of its code.
//
//   ref_logits <model-dir> <out.f32> <len> [<len> ...]
//
// For every length n the prompt is tokens[i] = (i * 37 + 5 + (i * i) % 7) % vocab, i < n (the
// same formula as tests/tiny.py's prompt(name, n, salt=0)), fed whole in one step from position 0;
// the logits of its last position are appended to the output as little-endian float32.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <vector>

#include "backend/backend.h"
#include "models/model.h"

int main(int argc, char** argv) {
    if (argc < 4) {
        std::fprintf(stderr, "usage: ref_logits <model-dir> <out.f32> <len>...\n");
        return 2;
    }
    using namespace xs;
    auto model = load_model(argv[1]);
    SessionOptions so;
    so.precision = DType::F32;
    so.max_context = 1024;
    auto session = make_backend("cpu-ref")->compile(model->graph(), model->weights(), so);
    const int64_t vocab = model->info().vocab_size;
    std::ofstream out(argv[2], std::ios::binary);
    for (int a = 3; a < argc; ++a) {
        const int n = std::atoi(argv[a]);
        std::vector<int32_t> prompt;
        for (int i = 0; i < n; ++i) prompt.push_back(static_cast<int32_t>((i * 37 + 5 + (i * i) % 7) % vocab));
        session->reset();
        TensorMap in, res;
        model->prepare_inputs(prompt, 0, {}, in);
        session->run(in, res);
        const float* logits = res.at("logits").data<float>();
        out.write(reinterpret_cast<const char*>(logits), static_cast<std::streamsize>(vocab * sizeof(float)));
        std::printf("len %d: argmax %d\n", n, res.at("argmax").data<int32_t>()[0]);
    }
    return 0;
}
