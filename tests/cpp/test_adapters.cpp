// Exercises the C++ protocol adapters over the C ABI on a GPU: forward() through ModelProtocol twice equals
// two steps through the handle; KernelProtocol::launch(); ComponentProtocol round trip.  Prints "ok" and exits 0.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "slime_pseudopod.hpp"

static float frand(unsigned& s) { s = s * 1664525u + 1013904223u; return (s >> 8) * (1.0f / 16777216.0f); }

int main() {
    const int B = 2, H = 16, W = 16, n = B * H * W * 64;
    unsigned seed = 7;
    std::vector<float> Wp(8 * 64 * 64), Wi(Wp.size()), Wv(Wp.size()), Wo(512 * 64), K(72, 1.f / 9.f), mu(8, 0.2f), sg(8, 0.03f), x(n);
    for (auto& v : Wp) v = (frand(seed) - 0.5f) * 0.4f;
    for (auto& v : Wi) v = (frand(seed) - 0.5f) * 0.4f;
    for (auto& v : Wv) v = (frand(seed) - 0.5f) * 0.4f;
    for (auto& v : Wo) v = (frand(seed) - 0.5f) * 0.15f;
    for (auto& v : x) v = frand(seed);
    try {
        SlimePseudopod pod(B, H, W);
        pod.set_weights(0, Wp.data(), Wi.data(), Wv.data(), Wo.data(), K.data(), mu.data(), sg.data());
        ModelProtocol* model = &pod;
        float *d_in, *d_mid, *d_out;
        cudaMalloc(&d_in, n * 4); cudaMalloc(&d_mid, n * 4); cudaMalloc(&d_out, n * 4);
        cudaMemcpy(d_in, x.data(), n * 4, cudaMemcpyHostToDevice);
        model->forward(d_in, d_mid);
        model->forward(d_mid, d_out);
        {
            // the documented protocol path: two chained forwards, then the component's fitness, with no launch() between
            SlimeComponent chained(&pod, 1);
            ComponentProtocol* c0 = &chained;
            const float f0 = c0->compute_fitness();
            if (!(f0 == f0) || !(std::fabs(f0 - model->effective_rank() * model->coherence()) < 1e-3f)) {
                std::printf("forward -> compute_fitness: f=%g\n", f0);
                return 1;
            }
        }
        std::vector<float> a(n), b(n);
        cudaMemcpy(a.data(), d_out, n * 4, cudaMemcpyDeviceToHost);
        // same two steps through KernelProtocol
        slime_ca_set_state(pod.handle(), x.data(), SLIME_CA_F32, nullptr);
        SlimeStepKernel kern(&pod, 2);
        KernelProtocol* kp = &kern;
        kp->launch();
        slime_ca_get_state(pod.handle(), b.data(), SLIME_CA_F32, nullptr);
        double num = 0, den = 0;
        for (int i = 0; i < n; ++i) { num += (double)(a[i] - b[i]) * (a[i] - b[i]); den += (double)b[i] * b[i]; }
        if (!(std::sqrt(num / den) < 1e-5)) { std::printf("forward twice != two steps: %g\n", std::sqrt(num / den)); return 1; }
        const float occ = kp->theoretical_occupancy();    // fp32 path: 256-thread CTAs, at least one and at most eight per SM
        if (kp->memory_required() == 0 || !(occ >= 256.f / 2048.f && occ <= 1.f)) { std::printf("kernel protocol: occupancy %g\n", occ); return 1; }
        SlimeComponent comp(&pod, 5);
        ComponentProtocol* cp = &comp;
        const float f = cp->compute_fitness();
        if (!(std::fabs(f - model->effective_rank() * model->coherence()) < 1e-3f) || !(std::fabs(cp->hunger - (1.f - cp->coherence)) < 1e-5f)) {
            std::printf("fitness bookkeeping: f=%g rank=%g coh=%g\n", f, model->effective_rank(), model->coherence());
            return 1;
        }
        char buf[128];
        cp->to_dict(buf);
        SlimeComponent other(&pod, 0);
        other.from_dict(buf);
        if (other.id != 5 || std::fabs(other.fitness - cp->fitness) > 1e-6f) { std::printf("dict round trip\n"); return 1; }
        cudaFree(d_in); cudaFree(d_mid); cudaFree(d_out);
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 1;
    }
    std::printf("ok\n");
    return 0;
}
