// Starts the reference's OWN engine (src/engine.cu, unmodified) on a model file and runs what its test calls
// "graph versus stream parity" (tests/test_kernels.cu:634-684): a prefill of eight tokens followed by fifteen
// greedy decode steps, once with the decode pass issued eagerly on the stream and once by replaying the CUDA
// graph the engine captured at start-up.  Linked against libw4a16_b200.so through dropin/w4a16_link_shim.cu,
// every W4 projection of those passes -- eager call, stream capture, graph replay -- is this library's.
// Prints both token rows; exit code 0 when all tokens lie in the vocabulary and the two rows are equal.
// Test infrastructure (built by `make -C oracle dropin`); not part of the product library.
#include <cstdio>
#include <exception>
#include <string>
#include <vector>

#include "config.cuh"
#include "tensor.cuh"
#include "engine.cuh"

int main(int argc, char** argv) {
    if (argc < 2) {
        std::fprintf(stderr, "usage: %s model.qwenbin\n", argv[0]);
        return 2;
    }
    constexpr int kSteps = 16;
    try {
        qwen::QwenEngine engine{std::string(argv[1])};
        const std::vector<int32_t> prompt = {9707, 11, 1246, 525, 498, 3351, 30, 220};
        std::vector<int32_t> eager, replay;

        engine.reset_session();
        eager.push_back(engine.prefill(prompt, 0.0f));
        for (int i = 1; i < kSteps; ++i) {
            engine.execute_decode_pass();
            if (cudaStreamSynchronize(engine.stream()) != cudaSuccess) return 3;
            eager.push_back(*engine.pinned_token_ptr());
        }
        engine.reset_session();
        replay.push_back(engine.prefill(prompt, 0.0f));
        for (int i = 1; i < kSteps; ++i) replay.push_back(engine.decode_step());

        bool ok = true;
        std::printf("EAGER ");
        for (int32_t t : eager) { std::printf(" %d", t); ok = ok && t >= 0 && t < qwen::VOCAB_SIZE; }
        std::printf("\nGRAPH ");
        for (int32_t t : replay) { std::printf(" %d", t); ok = ok && t >= 0 && t < qwen::VOCAB_SIZE; }
        int same = 0;
        for (int i = 0; i < kSteps; ++i) same += eager[i] == replay[i];
        std::printf("\nPARITY %d / %d\n", same, kSteps);
        return ok && same == kSteps ? 0 : 1;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "engine failed: %s\n", e.what());
        return 4;
    }
}
