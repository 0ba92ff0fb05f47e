// TEST INFRASTRUCTURE ONLY.  Times the reference's own three CA kernels (multi_head_ca_kernel,
// flow_lenia_dynamics_kernel, mix_heads_kernel; slime/core/pseudopod.cu:41-253), compiled from the reference tree
// where it lies, launched from the host once per repetition in the order and with the launch dimensions of the
// reference's step driver (slime/core/organism.cu:629-669), on weights from the reference's own initialisation kernel.
// One sequence, not the 128 concurrent ones the reference's driver starts.  Prints one JSON line with the
// CUDA-event time of each kernel averaged over the repetitions.  Context for the measured results only: the
// reference's step is a different function from the contract step (it computes 2 048 of its 16 384 cells and reads
// uninitialised shared memory), so nothing is compared with its output.
//
//   make -C oracle ref_step REFERENCE=<checkout of J0pari/Slime>     ->  oracle/_ref/ref_step
#include <cstdio>
#include <cstdlib>
#include <vector>

#include REF_PSEUDOPOD_CU   // the reference's slime/core/pseudopod.cu, path given by the Makefile

int main(int argc, char** argv) {
    const int reps = argc > 1 ? std::atoi(argv[1]) : 20;
    const size_t n_big = (size_t)NUM_HEADS * CHANNELS * HIDDEN_DIM, n_state = (size_t)GRID_SIZE * GRID_SIZE * CHANNELS;
    MultiHeadCAState hs{};
    cudaMalloc(&hs.perception_weights, n_big * 4); cudaMalloc(&hs.interaction_weights, n_big * 4);
    cudaMalloc(&hs.value_weights, n_big * 4); cudaMalloc(&hs.head_mixing_weights, 64 * 4);
    cudaMalloc(&hs.flow_kernels, 72 * 4); cudaMalloc(&hs.mass_buffer, 8 * 4);
    cudaMalloc(&hs.ca_input, n_state * 4); cudaMalloc(&hs.ca_output, n_state * 4);
    cudaMemset(hs.mass_buffer, 0, 8 * 4);
    MultiHeadCAState* d_state;
    cudaMalloc(&d_state, sizeof(hs));
    cudaMemcpy(d_state, &hs, sizeof(hs), cudaMemcpyHostToDevice);
    init_multihead_ca_kernel<<<(NUM_HEADS * CHANNELS * HIDDEN_DIM + 255) / 256, 256>>>(d_state, 1234u);
    std::vector<float> x(n_state);
    unsigned s = 42;
    for (auto& v : x) { s = s * 1664525u + 1013904223u; v = (s >> 8) * (1.0f / 16777216.0f) / (GRID_SIZE * GRID_SIZE); }
    cudaMemcpy(hs.ca_input, x.data(), n_state * 4, cudaMemcpyHostToDevice);
    cudaMemset(hs.ca_output, 0, n_state * 4);
    if (cudaDeviceSynchronize() != cudaSuccess) { std::fprintf(stderr, "setup failed\n"); return 1; }

    const dim3 init_grid((GRID_SIZE + 15) / 16, (GRID_SIZE + 15) / 16), init_block(16, 16);
    const dim3 ca_grid(GRID_SIZE / 16, NUM_HEADS, 1), ca_block(16, 16, 1);
    cudaEvent_t ev[4];
    for (auto& e : ev) cudaEventCreate(&e);
    double ms[3] = {0, 0, 0};
    for (int r = -3; r < reps; ++r) {
        cudaEventRecord(ev[0]);
        multi_head_ca_kernel<<<ca_grid, ca_block>>>(hs.ca_input, hs.perception_weights, hs.interaction_weights,
                                                    hs.value_weights, hs.ca_output, 1, GRID_SIZE);
        cudaEventRecord(ev[1]);
        flow_lenia_dynamics_kernel<<<init_grid, init_block>>>(hs.ca_input, hs.ca_output, hs.flow_kernels, hs.mass_buffer,
                                                              GRID_SIZE, 0.1f);
        cudaEventRecord(ev[2]);
        mix_heads_kernel<<<init_grid, init_block>>>(hs.ca_output, hs.head_mixing_weights, hs.ca_input, 1, GRID_SIZE);
        cudaEventRecord(ev[3]);
        const cudaError_t e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { std::fprintf(stderr, "%s\n", cudaGetErrorString(e)); return 1; }
        if (r >= 0)
            for (int k = 0; k < 3; ++k) { float t; cudaEventElapsedTime(&t, ev[k], ev[k + 1]); ms[k] += t; }
    }
    const double total = (ms[0] + ms[1] + ms[2]) / reps;
    std::printf("{\"reps\":%d,\"flags\":\"%s\",\"ms_multi_head_ca\":%.4f,\"ms_flow_lenia\":%.4f,\"ms_mix_heads\":%.4f,"
                "\"ms_sequence\":%.4f,\"cells_nominal\":%d,\"cells_computed_by_multi_head_ca\":%d,"
                "\"nominal_cell_updates_per_s\":%.1f}\n",
                reps, REF_FLAGS, ms[0] / reps, ms[1] / reps, ms[2] / reps, total, GRID_SIZE * GRID_SIZE,
                (GRID_SIZE / 16) * 16 * 16, GRID_SIZE * GRID_SIZE / (total * 1e-3));
    return 0;
}
