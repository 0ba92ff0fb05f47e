// TEST INFRASTRUCTURE ONLY.  Runs the reference's own create_elite_kernel (slime/memory/archive.cu:66-82), compiled
// from the reference tree where it lies, on seeded genomes and prints the GPUElite fields it fills (fitness,
// coherence, effective_rank, genome_hash, generation) with the genome as raw bit patterns.  The kernel reads
// genome[0 .. size) and writes one record from thread 0; nothing else.  The output is committed as a fixture: it
// pins the genome hash of this library's elite record (slime_ca_elite_record) to the reference's own arithmetic.
// Nothing in the product includes this file.
//
//   make -C oracle ref_elite REFERENCE=<checkout of J0pari/Slime>     ->  oracle/_ref/ref_elite
//   oracle/_ref/ref_elite > tests/golden/ref_elite.json
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include REF_ARCHIVE_CU   // the reference's slime/memory/archive.cu, path given by the Makefile

static uint32_t bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

int main() {
    const int sizes[4] = {1, 7, 64, 1000};
    unsigned s = 99;
    std::printf("{\"flags\":\"%s\",\"cases\":[", REF_FLAGS);
    for (int c = 0; c < 4; ++c) {
        const int n = sizes[c];
        std::vector<float> genome(n);
        for (auto& v : genome) { s = s * 1664525u + 1013904223u; v = ((float)(s >> 8) * (1.0f / 16777216.0f) - 0.5f) * 4.0f; }
        if (n > 2) { genome[1] = 0.0f; genome[2] = -0.0f; }
        const uint16_t gen = (uint16_t)(40 + 1000 * c);
        cudaMemcpyToSymbol(d_generation_counter, &gen, sizeof(gen));
        float* d_g;
        GPUElite* d_e;
        cudaMalloc(&d_g, n * 4); cudaMalloc(&d_e, sizeof(GPUElite));
        cudaMemset(d_e, 0, sizeof(GPUElite));
        cudaMemcpy(d_g, genome.data(), n * 4, cudaMemcpyHostToDevice);
        create_elite_kernel<<<1, 32>>>(d_e, d_g, 1.5f + c, 0.25f * c, 6.0f - c, (uint32_t)n);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { std::fprintf(stderr, "%s\n", cudaGetErrorString(e)); return 1; }
        GPUElite el;
        cudaMemcpy(&el, d_e, sizeof(el), cudaMemcpyDeviceToHost);
        std::printf("%s{\"genome\":[", c ? "," : "");
        for (int i = 0; i < n; ++i) std::printf("%s%u", i ? "," : "", bits(genome[i]));
        std::printf("],\"fitness\":%u,\"coherence\":%u,\"effective_rank\":%u,\"genome_hash\":\"%llu\",\"generation\":%u}",
                    bits(el.fitness), bits(el.coherence), bits(el.effective_rank), (unsigned long long)el.genome_hash,
                    (unsigned)el.generation);
        cudaFree(d_g); cudaFree(d_e);
    }
    std::printf("]}\n");
    return 0;
}
