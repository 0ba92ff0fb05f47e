// Exercises the source-level stand-in for slime/core/pseudopod.cu on a GPU: the kernels the reference's step
// driver launches are launched here from the host with the driver's own launch dimensions
// (slime/core/organism.cu:629-683), then slime_compat_generation() performs the recorded generation; the result
// must equal the same generation done through plain C-ABI calls.  Prints "ok" and exits 0.
#include <cmath>
#include <cstdio>
#include <vector>

#include "compat/pseudopod.cu"

#define CHECK(x) do { if (!(x)) { std::printf("failed: %s (line %d)\n", #x, __LINE__); return 1; } } while (0)

int main() {
    const size_t n_big = (size_t)NUM_HEADS * CHANNELS * HIDDEN_DIM, n_field = (size_t)GRID_SIZE * GRID_SIZE;
    MultiHeadCAState hs{};
    cudaMalloc(&hs.perception_weights, n_big * 4); cudaMalloc(&hs.interaction_weights, n_big * 4);
    cudaMalloc(&hs.value_weights, n_big * 4); cudaMalloc(&hs.head_mixing_weights, 64 * 4);
    cudaMalloc(&hs.flow_kernels, 72 * 4); cudaMalloc(&hs.mass_buffer, 8 * 4);
    cudaMalloc(&hs.ca_input, n_field * CHANNELS * 4); cudaMalloc(&hs.ca_output, n_field * CHANNELS * 4);
    MultiHeadCAState* d_state; cudaMalloc(&d_state, sizeof(hs));
    cudaMemcpy(d_state, &hs, sizeof(hs), cudaMemcpyHostToDevice);
    init_multihead_ca_kernel<<<(int)((n_big + 255) / 256), 256>>>(d_state, 1234u);
    CHECK(cudaDeviceSynchronize() == cudaSuccess);

    // the flow kernels are normalised, the mixing matrix is close to the identity
    std::vector<float> flow(72), mix(64);
    cudaMemcpy(flow.data(), hs.flow_kernels, 72 * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(mix.data(), hs.head_mixing_weights, 64 * 4, cudaMemcpyDeviceToHost);
    for (int h = 0; h < 8; ++h) { float s = 0; for (int t = 0; t < 9; ++t) s += flow[h * 9 + t]; CHECK(std::fabs(s - 1.f) < 1e-5f); }
    for (int i = 0; i < 64; ++i) CHECK(std::fabs(mix[i] - (i / 8 == i % 8 ? 1.f : 0.f)) < 0.1f);

    std::vector<float> field(n_field), lift(64), mu(8, 0.02f), sigma(8, 0.05f);
    unsigned s = 99;
    for (auto& v : field) { s = s * 1664525u + 1013904223u; v = 0.25f + (s >> 8) * (0.5f / 16777216.0f); }
    for (int c = 0; c < 64; ++c) lift[c] = 0.5f + 0.01f * c;
    float *d_field, *d_field2, *d_rank;
    cudaMalloc(&d_field, n_field * 4); cudaMalloc(&d_field2, n_field * 4); cudaMalloc(&d_rank, 16 * 4);
    cudaMemcpy(d_field, field.data(), n_field * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(d_field2, field.data(), n_field * 4, cudaMemcpyHostToDevice);
    cudaMemset(d_rank, 0, 16 * 4);

    for (int dtype : {SLIME_CA_F32, SLIME_CA_BF16}) {
        slime_ca* ca = nullptr;
        CHECK(slime_compat_bind(&ca, d_state, dtype, mu.data(), sigma.data()) == SLIME_CA_OK);
        CHECK(slime_compat_generation(ca, d_field, lift.data(), 2, nullptr) == 0);   // nothing was requested yet

        // the launch sites of the reference's step driver, with its dimensions
        dim3 init_grid((GRID_SIZE + 15) / 16, (GRID_SIZE + 15) / 16), init_block(16, 16);
        dim3 ca_grid(GRID_SIZE / 16, NUM_HEADS, 1), ca_block(16, 16, 1);
        multi_head_ca_kernel<<<ca_grid, ca_block>>>(hs.ca_input, hs.perception_weights, hs.interaction_weights,
                                                    hs.value_weights, hs.ca_output, 1, GRID_SIZE);
        flow_lenia_dynamics_kernel<<<init_grid, init_block>>>(hs.ca_input, hs.ca_output, hs.flow_kernels, hs.mass_buffer, GRID_SIZE, 0.1f);
        mix_heads_kernel<<<init_grid, init_block>>>(hs.ca_output, hs.head_mixing_weights, hs.ca_input, 1, GRID_SIZE);
        compute_effective_rank_kernel<<<1, 256>>>(hs.perception_weights, d_rank + 3, (int)n_big);
        CHECK(cudaDeviceSynchronize() == cudaSuccess);
        CHECK(slime_compat_generation(ca, d_field, lift.data(), 2, nullptr) == 1);
        CHECK(slime_compat_generation(ca, d_field, lift.data(), 2, nullptr) == 0);   // the request was consumed

        float rank = 0.f;
        cudaMemcpy(&rank, d_rank + 3, 4, cudaMemcpyDeviceToHost);
        CHECK(rank >= 1.f && rank <= 64.f);

        // the same generation through plain C-ABI calls on a second handle
        slime_ca* cb = nullptr;
        CHECK(slime_compat_bind(&cb, d_state, dtype, mu.data(), sigma.data()) == SLIME_CA_OK);
        CHECK(slime_ca_lift_field_device(cb, d_field2, lift.data(), nullptr) == SLIME_CA_OK);
        CHECK(slime_ca_step(cb, 2, nullptr) == SLIME_CA_OK);
        CHECK(slime_ca_field_from_state_device(cb, d_field2, nullptr) == SLIME_CA_OK);
        CHECK(cudaDeviceSynchronize() == cudaSuccess);
        std::vector<float> a(n_field), b(n_field);
        cudaMemcpy(a.data(), d_field, n_field * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(b.data(), d_field2, n_field * 4, cudaMemcpyDeviceToHost);
        double moved = 0;
        for (size_t i = 0; i < n_field; ++i) {
            CHECK(std::isfinite(a[i]));
            CHECK(a[i] == b[i]);
            moved += std::fabs(a[i] - field[i]);
        }
        CHECK(moved > 0);
        slime_ca_destroy(ca); slime_ca_destroy(cb);
        // next dtype starts from the original field
        cudaMemcpy(d_field, field.data(), n_field * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(d_field2, field.data(), n_field * 4, cudaMemcpyHostToDevice);
    }
    std::printf("ok\n");
    return 0;
}
