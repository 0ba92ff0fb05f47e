// TEST INFRASTRUCTURE ONLY.  Runs the reference's own weight-initialisation kernel (init_multihead_ca_kernel,
// slime/core/pseudopod.cu:386-444), compiled from the reference tree where it lies, with the reference's own
// launch dimensions (slime/core/organism.cu:926-929), and prints a fingerprint of every array it fills as one
// JSON object: element count, the first 16 values as raw bit patterns, and two order-independent checksums
// (wrapping sum and XOR of all bit patterns).  The output is committed as a fixture; the stand-in for that
// kernel (include/compat/pseudopod.cu) is compared with it.  Nothing in the product includes this file.
//
//   make -C oracle ref_init REFERENCE=<checkout of J0pari/Slime>     ->  oracle/_ref/ref_init
//   oracle/_ref/ref_init 1234 > tests/golden/ref_init_seed1234.json
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include REF_PSEUDOPOD_CU   // the reference's slime/core/pseudopod.cu, path given by the Makefile

static void fingerprint(const char* name, const float* dev, size_t n, bool last) {
    std::vector<uint32_t> h(n);
    cudaMemcpy(h.data(), dev, n * sizeof(float), cudaMemcpyDeviceToHost);
    uint64_t sum = 0;
    uint32_t x = 0;
    for (size_t i = 0; i < n; ++i) { sum += h[i]; x ^= h[i]; }
    std::printf("\"%s\":{\"n\":%zu,\"sum\":%llu,\"xor\":%u,\"first\":[", name, n, (unsigned long long)sum, x);
    for (size_t i = 0; i < 16 && i < n; ++i) std::printf("%s%u", i ? "," : "", h[i]);
    std::printf("]}%s", last ? "" : ",");
}

int main(int argc, char** argv) {
    const unsigned seed = argc > 1 ? (unsigned)std::strtoul(argv[1], nullptr, 10) : 1234u;
    const size_t n_big = (size_t)NUM_HEADS * CHANNELS * HIDDEN_DIM;
    MultiHeadCAState hs{};
    cudaMalloc(&hs.perception_weights, n_big * 4); cudaMalloc(&hs.interaction_weights, n_big * 4);
    cudaMalloc(&hs.value_weights, n_big * 4); cudaMalloc(&hs.head_mixing_weights, 64 * 4);
    cudaMalloc(&hs.flow_kernels, 72 * 4); cudaMalloc(&hs.mass_buffer, 8 * 4);
    hs.ca_input = hs.ca_output = nullptr;
    MultiHeadCAState* d_state;
    cudaMalloc(&d_state, sizeof(hs));
    cudaMemcpy(d_state, &hs, sizeof(hs), cudaMemcpyHostToDevice);
    init_multihead_ca_kernel<<<(NUM_HEADS * CHANNELS * HIDDEN_DIM + 255) / 256, 256>>>(d_state, seed);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { std::fprintf(stderr, "%s\n", cudaGetErrorString(e)); return 1; }
    std::printf("{\"seed\":%u,\"flags\":\"%s\",", seed, REF_FLAGS);
    fingerprint("perception_weights", hs.perception_weights, n_big, false);
    fingerprint("interaction_weights", hs.interaction_weights, n_big, false);
    fingerprint("value_weights", hs.value_weights, n_big, false);
    fingerprint("head_mixing_weights", hs.head_mixing_weights, 64, false);
    // all 72 taps: the reference normalises them with a cross-thread read that nothing orders
    {
        std::vector<uint32_t> h(72);
        cudaMemcpy(h.data(), hs.flow_kernels, 72 * 4, cudaMemcpyDeviceToHost);
        std::printf("\"flow_kernels\":{\"n\":72,\"all\":[");
        for (int i = 0; i < 72; ++i) std::printf("%s%u", i ? "," : "", h[i]);
        std::printf("]}");
    }
    std::printf("}\n");
    return 0;
}
