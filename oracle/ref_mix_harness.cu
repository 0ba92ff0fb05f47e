// TEST INFRASTRUCTURE ONLY.  Runs the reference's own mix_heads_kernel (slime/core/pseudopod.cu:217-253), compiled
// from the reference tree where it lies, with the launch dimensions of the reference's step driver
// (slime/core/organism.cu:629-630,663-669) on seeded head outputs, and prints - as raw bit patterns - the 8 x 8
// mixing matrix and, for a few sample cells, the kernel's inputs [8 heads][64] and outputs [512].  The output is
// committed as a fixture: it pins how this library folds the reference's head mixing into the contract's output
// projection (slime_ca_set_weights_reference_layout).  Nothing in the product includes this file.
//
//   make -C oracle ref_mix REFERENCE=<checkout of J0pari/Slime>     ->  oracle/_ref/ref_mix
//   oracle/_ref/ref_mix > tests/golden/ref_mix_heads.json
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include REF_PSEUDOPOD_CU   // the reference's slime/core/pseudopod.cu, path given by the Makefile

static uint32_t bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

int main() {
    const int G = GRID_SIZE;
    const size_t n = (size_t)NUM_HEADS * G * G * HEAD_DIM;
    std::vector<float> in(n), mix(NUM_HEADS * NUM_HEADS), out(n);
    unsigned s = 2024;
    for (auto& v : in) { s = s * 1664525u + 1013904223u; v = (float)(s >> 8) * (1.0f / 16777216.0f) - 0.5f; }
    for (int i = 0; i < NUM_HEADS * NUM_HEADS; ++i) {
        s = s * 1664525u + 1013904223u;
        mix[i] = (i / NUM_HEADS == i % NUM_HEADS ? 1.0f : 0.0f) + 0.25f * ((float)(s >> 8) * (1.0f / 16777216.0f) - 0.5f);
    }
    float *d_in, *d_mix, *d_out;
    cudaMalloc(&d_in, n * 4); cudaMalloc(&d_mix, mix.size() * 4); cudaMalloc(&d_out, n * 4);
    cudaMemcpy(d_in, in.data(), n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_mix, mix.data(), mix.size() * 4, cudaMemcpyHostToDevice);
    const dim3 grid((G + 15) / 16, (G + 15) / 16), block(16, 16);
    mix_heads_kernel<<<grid, block>>>(d_in, d_mix, d_out, 1, G);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { std::fprintf(stderr, "%s\n", cudaGetErrorString(e)); return 1; }
    cudaMemcpy(out.data(), d_out, n * 4, cudaMemcpyDeviceToHost);
    std::printf("{\"flags\":\"%s\",\"grid\":%d,\"mixing\":[", REF_FLAGS, G);
    for (size_t i = 0; i < mix.size(); ++i) std::printf("%s%u", i ? "," : "", bits(mix[i]));
    std::printf("],\"cells\":[");
    const int cells[6][2] = {{0, 0}, {127, 127}, {5, 77}, {64, 1}, {33, 126}, {100, 50}};   // (y, x)
    for (int c = 0; c < 6; ++c) {
        const int y = cells[c][0], x = cells[c][1];
        std::printf("%s{\"y\":%d,\"x\":%d,\"head_outputs\":[", c ? "," : "", y, x);
        for (int h = 0; h < NUM_HEADS; ++h)
            for (int d = 0; d < HEAD_DIM; ++d)      // [head][y][x][d], the layout the kernel reads (pseudopod.cu:236-239)
                std::printf("%s%u", (h || d) ? "," : "", bits(in[(((size_t)h * G + y) * G + x) * HEAD_DIM + d]));
        std::printf("],\"final_output\":[");
        for (int k = 0; k < CHANNELS; ++k)           // [y][x][512], out_head * 64 + c (pseudopod.cu:244-249)
            std::printf("%s%u", k ? "," : "", bits(out[((size_t)y * G + x) * CHANNELS + k]));
        std::printf("]}");
    }
    std::printf("]}\n");
    return 0;
}
