/*
 * slime_ca.h - C ABI of the B200 (sm_100a) multi-head Flow-Lenia neural-CA step.
 *
 * This is the boundary a J0pari/Slime maintainer binds instead of the CA kernels of
 * slime/core/pseudopod.cu and their device-side driver in slime/core/organism.cu.  Plain pointers and sizes
 * only; every call returns an int status (0 = ok) and never exits the process (the reference's CUDA_CHECK,
 * slime/runtime.cu:11-20, prints and calls exit(1)).
 *
 * One handle drives one GPU.  A handle owns its state, intermediates and workspace; the caller owns every
 * pointer it passes in.  slime_ca_step() allocates nothing.  Calls on one handle must not overlap; different
 * handles are independent.  `stream` arguments are a cudaStream_t passed as void* (NULL = default stream).
 */
#ifndef SLIME_CA_H
#define SLIME_CA_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SLIME_CA_NUM_HEADS 8   /* slime/core/pseudopod.cu:15 NUM_HEADS */
#define SLIME_CA_HEAD_DIM 64   /* slime/core/pseudopod.cu:16 HEAD_DIM  */
#define SLIME_CA_CHANNELS 64   /* channels of the state the step reads and writes */

enum slime_ca_status {
    SLIME_CA_OK = 0,
    SLIME_CA_EINVAL = 1,  /* bad argument (null pointer, bad shape, index out of range)          */
    SLIME_CA_ECUDA = 2,   /* a CUDA runtime call failed; slime_ca_last_error() has the text       */
    SLIME_CA_ENOMEM = 3,  /* host or device allocation failed                                     */
    SLIME_CA_ESTATE = 4,  /* call order: weights or state not set, fitness before two steps, ...  */
    SLIME_CA_EDEVICE = 5, /* a kernel reported an error through its status word (bounded wait ran out);    */
                          /* the state is undefined afterwards: load it again before further steps          */
    SLIME_CA_ECOMM = 6,   /* the row-stripe ring's communicator (NCCL) failed or could not be loaded          */
    SLIME_CA_ETIMEOUT = 7 /* slime_ca_ring_wait: the stream did not drain before the deadline               */
};

enum slime_ca_dtype {
    SLIME_CA_F32 = 0,  /* fp32 storage and arithmetic (SIMT)                                             */
    SLIME_CA_BF16 = 1  /* bf16 storage of state/weights/intermediates, fp32 accumulate, tcgen05 projections */
};

enum slime_ca_buffer {
    SLIME_CA_BUF_STATE = 0,       /* [batch][height + 2*halo][width][64], dtype of the handle, un-normalised */
    SLIME_CA_BUF_SCALE = 1,       /* [batch][64] fp32: true state = stored state * scale                     */
    SLIME_CA_BUF_MASS = 2,        /* [batch][64] fp64: target per-channel masses                             */
    SLIME_CA_BUF_SUMS = 3,        /* [batch][64] fp64: per-channel sums of the stored state's own rows       */
    SLIME_CA_BUF_VPRIME_PREV = 4, /* [batch][8][height][width][64]: redistributed value of step n-1         */
    SLIME_CA_BUF_VPRIME_LAST = 5  /* same, step n                                                            */
};

/*
 * Replaces the fixed constexpr configuration of slime/core/pseudopod.cu:15-21 (GRID_SIZE = 128, batch 1).
 */
typedef struct slime_ca_config {
    int batch;          /* independent grids held by this handle                                          */
    int height;         /* rows per grid owned by this handle                                             */
    int width;          /* columns per grid                                                               */
    int n_weight_sets;  /* grid b uses weight set b / (batch / n_weight_sets); must divide batch           */
    int dtype;          /* enum slime_ca_dtype                                                            */
    float dt;           /* residual step size; the reference uses 0.1 (slime/core/organism.cu:659)        */
    int device;         /* CUDA device ordinal                                                            */
    int stripe;         /* 0: every grid is a full torus.  1: the grid is a row stripe of a taller torus:  */
                        /*    the state buffer carries 3 halo rows above and below the `height` own rows,  */
                        /*    which the caller refreshes before every step (x still wraps)                 */
    int keep_vprime;    /* 1: keep the redistributed value V' of the last two steps (needed by fitness)    */
} slime_ca_config;

typedef struct slime_ca slime_ca;

/* Handle lifetime.  Replaces the CA part of create_organism()/destroy_organism() (slime/runtime.cu:26,417:
 * cudaMalloc of weights, ca_input, ca_output, mass_buffer at slime/runtime.cu:66-94). */
int slime_ca_create(const slime_ca_config* cfg, slime_ca** out);
int slime_ca_destroy(slime_ca* h);

/* Text of the last failure on this handle (never NULL).  The reference has no status channel. */
const char* slime_ca_last_error(const slime_ca* h);

/* Device bytes the handle holds (state + intermediates + workspace).  Backs KernelProtocol::memory_required()
 * (slime/proto/kernel.cu:13). */
size_t slime_ca_workspace_bytes(const slime_ca* h);

/*
 * Upload one weight set from HOST fp32 arrays in the reference's index order (slime/core/pseudopod.cu:86-87):
 *   Wp, Wi, Wv [8][64][64] = [head][c_in][d_out];  Wo [512][64] = [head*64+d][c_out];
 *   K [8][9] taps t=(dy+1)*3+(dx+1) (slime/core/pseudopod.cu:153);  mu, sigma [8] growth centre and width.
 * Replaces init_multihead_ca_kernel (slime/core/pseudopod.cu:386-444) as the way weights reach the device.
 * Waits for the device to drain first (cudaDeviceSynchronize): steps in flight on any stream read the arrays this
 * call overwrites.  Uploads run on the default stream and the call returns with them complete.
 */
int slime_ca_set_weights(slime_ca* h, int set_index, const float* Wp, const float* Wi, const float* Wv,
                         const float* Wo, const float* K, const float* mu, const float* sigma);

/*
 * Load / read the state from HOST memory, [batch][height][width][64] in `host_dtype` (fp32 or bf16).
 * set_state also records each (grid, channel) sum as its target mass.  get_state returns the normalised
 * state (stored state * scale).  Replaces initialize_ca_from_field / get_ca_state as the way state enters
 * and leaves (slime/core/organism.cu:691-720, slime/runtime.cu:479-504).  Both synchronise `stream`.
 */
int slime_ca_set_state(slime_ca* h, const void* host_state, int host_dtype, void* stream);
int slime_ca_get_state(slime_ca* h, void* host_state, int host_dtype, void* stream);

/* Same with DEVICE pointers (no synchronisation).  A caller that never synchronises through this library
 * (set_state_device / step / get_state_device on its own stream) still learns of a kernel that gave up on a
 * bounded wait: every batch of steps copies the status word back to pinned host memory behind itself, and
 * slime_ca_step, slime_ca_step_partial, slime_ca_step_ring and slime_ca_get_state_device return
 * SLIME_CA_EDEVICE at their next call once that copy has run.  set_state_device clears the condition. */
int slime_ca_set_state_device(slime_ca* h, const void* dev_state, int dtype, void* stream);
int slime_ca_get_state_device(slime_ca* h, void* dev_state, int dtype, void* stream);

/* Override / read the target masses, HOST fp64 [batch][64] (stripe mode: the caller supplies global sums). */
int slime_ca_set_mass(slime_ca* h, const double* mass);
int slime_ca_get_mass(slime_ca* h, double* mass);

/*
 * n_steps of the CA step on every grid of the handle, enqueued on `stream`; returns without synchronising.
 * Replaces neural_ca_update_kernel and the three kernels it launches (slime/core/organism.cu:617-688;
 * slime/core/pseudopod.cu:41-131, 134-214, 217-253).
 */
int slime_ca_step(slime_ca* h, int n_steps, void* stream);

/*
 * Stripe mode, several ranks: one step split around the caller's all-reduce.
 *   slime_ca_step_partial  runs the step's kernels and leaves this rank's per-channel sums in BUF_SUMS;
 *   (caller sums BUF_SUMS over ranks, e.g. ncclAllReduce, and refreshes the halo rows of BUF_STATE)
 *   slime_ca_step_finish   turns BUF_SUMS and BUF_MASS into the new BUF_SCALE.
 * slime_ca_step(h, 1, s) equals partial followed by finish.
 */
int slime_ca_step_partial(slime_ca* h, void* stream);
int slime_ca_step_finish(slime_ca* h, void* stream);

/*
 * Stripe mode, the ring inside the library: one torus split into row stripes, one handle (GPU, rank) per stripe,
 * ranks forming a ring in y.  The reference has no multi-GPU code (one line of intent, BLUEPRINT.md:444-447;
 * main.cu:12-13 selects device 0); this is the library's own answer for the large-grid workload.
 *   slime_ca_ring_unique_id   rank 0 makes the 128-byte id (ncclGetUniqueId) and ships it to the other ranks by any
 *                             means; slime_ca_ring_init(h, id, rank, world) is then called by every rank at the
 *                             same time (ncclCommInitRank).  world = 1 needs no id and no NCCL: the stripe wraps
 *                             onto itself.
 *   slime_ca_ring_attach      the same with the caller's own ncclComm_t (passed as void*), which is not destroyed
 *                             by the library.
 *   slime_ca_ring_sync_mass   after loading every rank's own rows: sums the target masses over the ranks, so that
 *                             each is the mass of the whole torus.
 *   slime_ca_step_ring        n_steps steps, each: grouped ncclSend / ncclRecv of the 3 + 3 halo rows straight between
 *                             the neighbours' state buffers, the step's kernels, ncclAllReduce of the 64 per-channel
 *                             sums (fp64) of every grid, the new scale.  All of it is enqueued on `stream`; nothing
 *                             synchronises with the host.  Kernels only ever read this GPU's own memory.
 *   slime_ca_step_ring_timed  the same with CUDA events: ms[0] halo exchange, ms[1] the step's kernels and the local
 *                             reduction, ms[2] all-reduce and scale, summed over the steps.  Synchronises.
 *   slime_ca_ring_wait        bounded host wait for `stream` to drain: polls the stream and the communicator's
 *                             asynchronous error state; on an NCCL error (SLIME_CA_ECOMM) or when timeout_ms runs out
 *                             (SLIME_CA_ETIMEOUT) it aborts the communicator (ncclCommAbort) so that the stream ends,
 *                             and the handle is left without a ring.  The reference's only error path is exit(1)
 *                             (slime/runtime.cu:11-20).
 * NCCL is bound at run time to the copy the process already carries, else to libnccl.so.2.
 */
#define SLIME_CA_RING_ID_BYTES 128
int slime_ca_ring_unique_id(void* id_out);
int slime_ca_ring_init(slime_ca* h, const void* id, int rank, int world);
int slime_ca_ring_attach(slime_ca* h, void* nccl_comm, int rank, int world);
int slime_ca_ring_detach(slime_ca* h);
int slime_ca_ring_sync_mass(slime_ca* h, void* stream);
int slime_ca_step_ring(slime_ca* h, int n_steps, void* stream);
int slime_ca_step_ring_timed(slime_ca* h, int n_steps, void* stream, float* ms);
int slime_ca_ring_wait(slime_ca* h, void* stream, int timeout_ms);

/*
 * Profiling aid with no counterpart in the reference: n_steps steps with CUDA events recorded on `stream`
 * around each kernel; ms[0..2] receive the summed device time of the projection/growth kernel, of the
 * redistribution/output kernel and of the reduction + scale kernels.  Synchronises `stream`.
 */
int slime_ca_step_timed(slime_ca* h, int n_steps, void* stream, float* ms);

/* Device address and size of one of the handle's buffers (enum slime_ca_buffer), for halo exchange,
 * all-reduce and zero-copy views.  The reference exposes raw device pointers in MultiHeadCAState
 * (slime/core/pseudopod.cu:29-38). */
int slime_ca_buffer(slime_ca* h, int which, void** dev_ptr, size_t* bytes);

/*
 * Fitness of every grid from V' of the last two steps (needs keep_vprime and at least two steps):
 * HOST fp32 arrays of `batch` elements, any of which may be NULL.  rank = mean over heads of the
 * exp-entropy rank of that head's 64x64 Gram spectrum (Jacobi), coherence = Pearson r between the two
 * steps, fitness = rank * coherence, hunger = 1 - coherence.  Replaces fitness_fused_kernel and its
 * children (slime/kernels/warp_ca.cu:66-226) and the hunger kernel (:229-240).  Synchronises `stream`.
 */
int slime_ca_fitness(slime_ca* h, float* rank, float* coherence, float* fitness, float* hunger, void* stream);

/* Read one weight set back (HOST fp32 arrays in the layouts of slime_ca_set_weights; any may be NULL): the
 * device-resident master copy, i.e. what was uploaded or what the population step made of it. */
int slime_ca_get_weights(slime_ca* h, int set_index, float* Wp, float* Wi, float* Wv, float* Wo, float* K, float* mu,
                         float* sigma);

/*
 * The population step that consumes the fitness scalars, on the device: replaces culling_kernel,
 * selection_kernel's search for the best, and spawn_wave_kernel / spawn_component_kernel
 * (slime/core/organism.cu:430-470,556-614; slime/memory/pool.cu:57-121) for a population of weight sets.
 *   fitness, hunger of a weight set = mean over its grids of the values slime_ca_fitness last computed;
 *   culled  : fitness < 0.1 * fitness_threshold, or hunger > hunger_threshold, or not finite
 *             (slime/core/organism.cu:594-611);
 *   best    : highest fitness among the survivors, lowest index on ties (slime/core/organism.cu:442-470);
 *   refill  : every culled set becomes a copy of the best whose Wp, Wi, Wv, Wo values are each perturbed with
 *             probability mutation_rate by mutation_sigma * N(0, 1) (slime/memory/pool.cu:84-93; the driver
 *             uses rate 0.01, slime/core/organism.cu:578); taps, mu and sigma are inherited unchanged.  If no
 *             set survives nothing changes.
 * The draws depend only on (seed, generation, set index, value index).  Must follow slime_ca_fitness on the same
 * state.  parent: HOST [n_weight_sets] or NULL, parent[s] = s for survivors, the best set for replaced ones;
 * best_set (-1 if none survived) and n_replaced may be NULL.  Synchronises `stream`.
 */
typedef struct slime_ca_evolve_params {
    float fitness_threshold;
    float hunger_threshold;
    float mutation_rate;
    float mutation_sigma;
    unsigned long long seed;
    int generation;
} slime_ca_evolve_params;
int slime_ca_evolve(slime_ca* h, const slime_ca_evolve_params* p, int* parent, int* best_set, int* n_replaced,
                    void* stream);

/* Lift a one-channel HOST image batch [batch][img_h][img_w] (fp32) into the state: zero-pad to
 * height x width (centred), X = pixel * L[c].  Mirrors initialize_ca_from_field_kernel
 * (slime/core/organism.cu:691-720). */
int slime_ca_lift_images(slime_ca* h, const float* host_img, int img_h, int img_w, const float* host_L,
                         void* stream);

/* Mean-pool the normalised state over space and apply a 64 -> n_out linear readout (HOST fp32 Wr[64][n_out],
 * br[n_out] or NULL) into HOST logits[batch][n_out].  The pooling mirrors update_field_from_ca_kernel
 * (slime/core/organism.cu:723-743). */
int slime_ca_pool_readout(slime_ca* h, const float* host_Wr, const float* host_br, int n_out,
                          float* host_logits, void* stream);

/* The same lift from a DEVICE field [batch][height][width] (fp32) of the grid's own size, as the reference's step
 * driver does every generation (initialize_ca_from_field_kernel, slime/core/organism.cu:632-636,691-720):
 * X = field * L[c] with HOST L[64]; the masses become those of the lifted state.  Synchronises `stream`. */
int slime_ca_lift_field_device(slime_ca* h, const float* dev_field, const float* host_L, void* stream);

/* Write the CA back into a DEVICE field [batch][height][width] (fp32): the mean over the 64 channels of each
 * cell of the normalised state.  Mirrors update_field_from_ca_kernel (slime/core/organism.cu:723-743).  Enqueued
 * on `stream`, not synchronised. */
int slime_ca_field_from_state_device(slime_ca* h, float* dev_field, void* stream);

/*
 * Upload one weight set straight from the reference's weight bundle (struct MultiHeadCAState,
 * slime/core/pseudopod.cu:29-38): DEVICE fp32 arrays perception [8][512][256], interaction [8][512][256],
 * value [8][256][512], head mixing [8][8], flow kernels [8][9].  Taken as the reference's kernels index them:
 * Wp, Wi = rows c < 64, columns d < 64 of each head's matrix (slime/core/pseudopod.cu:86-87,102-103);
 * Wv[c][d] = sum over r < 4 of value[c + 64 r][d] (the loop j < 256 with interaction[j % 64], :114-119);
 * K = flow kernels as stored; Wo[(h, d)][c] = (d == c) * mean over output heads o of mixing[o][h] (the 8 x 8
 * mixing of :231-249 followed by the mean of the output heads: the bundle has no 512 -> 64 projection).
 * mu, sigma: HOST [8], or NULL for 0.2 and 0.03 (the bundle carries none).
 */
int slime_ca_set_weights_reference_layout(slime_ca* h, int set_index, const float* dev_perception,
                                          const float* dev_interaction, const float* dev_value,
                                          const float* dev_head_mixing, const float* dev_flow_kernels,
                                          const float* mu, const float* sigma);

/*
 * One line of the reference's trajectory file evolution.json (extract_system_state, slime/extract_state.cu:58-184,
 * written every 100 generations by slime/runtime.cu:402-408) for one grid, into `buf` (NUL-terminated, `cap`
 * bytes; *written = length without the NUL, also when `cap` is too small, which returns SLIME_CA_EINVAL):
 *   {"gen":G,"elapsed":S.SS,"chemical":{"concentration":[16 x 16 centre sample, %.4f],"size":16},
 *    "ca":{"flow_kernels":[[9 x %.4f] x 8]},"agents":[],"voronoi":[],"archive":{"size":0,"elites":[]},
 *    "pool":{"active":A,"capacity":C,"spawned":S,"culled":K}}\n
 * with the reference's key order and number formats, so the two files can be read by the same tools.  The
 * concentration is sampled from `dev_field` (DEVICE [height][width] fp32) or, when NULL, from the channel mean of
 * the grid's normalised state; the flow kernels are those of the grid's weight set.  Agents, Voronoi cells and the
 * elite archive belong to subsystems outside this library and are written empty; the pool counters are the
 * caller's (e.g. from slime_ca_evolve).  Synchronises `stream`.
 */
int slime_ca_evolution_record(slime_ca* h, int grid_index, int generation, double elapsed_seconds,
                              const float* dev_field, int pool_active, int pool_capacity, int pool_spawned,
                              int pool_culled, char* buf, size_t cap, size_t* written, void* stream);

/*
 * The record the reference keeps of an elite (struct GPUElite, slime/memory/archive.cu:9-20, filled by
 * create_elite_kernel :66-82) for one weight set, after slime_ca_fitness (and, for the parents, slime_ca_evolve):
 * fitness, coherence and effective_rank are the means over the set's grids; genome_hash is the reference's hash
 * (gpu_sha256, archive.cu:41-60) over the set's 131 168 fp32 master weights in upload order
 * (Wp | Wi | Wv | Wo | K | mu | sigma); parent_ids name the set it was copied from at the last population step (itself
 * for a survivor; both slots the same, the refill has one parent); generation is truncated to 16 bits as in the
 * reference.  The behavioural coordinates, the compressed genome and the raw metrics of GPUElite belong to the
 * archive, outside this library.  Synchronises `stream`.
 */
typedef struct slime_ca_elite {
    float fitness;
    float coherence;
    float effective_rank;
    unsigned long long genome_hash;
    unsigned int parent_ids[2];
    unsigned short generation;
} slime_ca_elite;
int slime_ca_elite_record(slime_ca* h, int set_index, int generation, slime_ca_elite* out, void* stream);

/* Resident threads per SM of the step kernels of this handle's dtype over the SM's thread limit, from
 * cudaOccupancyMaxActiveBlocksPerMultiprocessor (the smaller of the two kernels).  Backs
 * KernelProtocol::theoretical_occupancy() (slime/proto/kernel.cu:14). */
int slime_ca_occupancy(slime_ca* h, float* occupancy);

/*
 * Self-test of the bounded device-side waits, with no counterpart in the reference: launches one thread that waits
 * `limit_ns` (at most 100 ms) on a barrier nobody arrives on, gives up, and records code 901 in the handle's status
 * word.  The next synchronising call on the handle (or the next step call, once the word has been copied back)
 * returns SLIME_CA_EDEVICE and clears the word; the context stays usable.
 */
int slime_ca_selftest_bounded_wait(slime_ca* h, unsigned long long limit_ns, void* stream);

/* Number of kernels the library has launched on this handle since creation (for launch accounting). */
long long slime_ca_launch_count(const slime_ca* h);

/*
 * The host launcher the reference planned but never wrote (buildplan.md:635-655):
 *   ca_state  device fp32 [batch][grid][grid][64]
 *   weights   device fp32 [P | I | V], each [8][64][64]
 *   ca_output device fp32 [batch][8][grid][grid][64]: each head's redistributed value V'
 * Flow kernels are uniform (1/9 per tap) and the growth uses mu = 0.2, sigma = 0.03, the midpoints of the
 * ranges the weights are drawn from, because the planned signature carries neither.  Runs on the default
 * stream and synchronises.  Returns nothing, as planned; errors are printed to stderr.
 * A shim: it keeps one handle in a function-local static (re-made when the shape or the device changes, never
 * freed), so it is not safe to call from two host threads at once, and it passes the weights through the host on
 * every call.  Code that steps repeatedly should hold a handle and call slime_ca_step.
 */
void launch_multi_head_ca(float* ca_state, float* weights, float* ca_output, int batch_size, int grid_size);

/*
 * Per-channel sums of a dense DEVICE state [batch][cells_per_grid][64] (fp32 or bf16) into DEVICE
 * dev_sums[batch][64] (fp64), computed without allocating anything.  No counterpart in the reference.
 *
 * For callers that can not call cudaMalloc where they need a state's channel masses: a host loop that has
 * given the whole device to its own memory pool (so a cudaMalloc fails), or a latency-critical loop that can
 * not take the device-wide synchronisation cudaMalloc / cudaFree imply.  This call makes no cudaMalloc, no
 * cudaFree and no allocating library call; its only scratch is a 2 MiB array built into the library image
 * (every GPU that loads the library holds it until the process exits).
 *
 * Limit: batch * ceil(cells_per_grid / 256) <= 8192 (at most 2 097 152 cells per call); larger requests return
 * SLIME_CA_EINVAL and slime_ca_static_error() says so.  The first call on each device resolves the address of
 * the built-in array; make that first call outside any stream capture, and make it early: once per device at
 * start-up, before a memory pool takes the device and before the hot loop, because with lazy module loading that
 * call may also be the one that loads the library's kernels and the array itself (which allocates and can
 * synchronise).  The resolved address is cached per device ordinal for the life of the process: it is stale
 * after cudaDeviceReset(), which this entry point does not survive.  Two host threads may make the first call on
 * one device at once (they store the same address).  All calls on a device share the array,
 * which keeps whatever the last call left: nothing needs to start at zero (every slot a call reads it has
 * written first), but two calls whose kernels overlap on the GPU (different streams, different host threads)
 * race on it - run them one after the other.  Work is enqueued on `stream` of the CURRENT device; no
 * synchronisation.  Same numbers as slime_ca_set_state_device + slime_ca_get_mass up to fp64 summation order.
 */
int slime_ca_channel_sums_static(const void* dev_state, int dtype, int batch, int cells_per_grid, double* dev_sums,
                                 void* stream);

/* Text of the last failure of slime_ca_channel_sums_static on the calling thread ("" after a success). */
const char* slime_ca_static_error(void);

#ifdef __cplusplus
}
#endif
#endif /* SLIME_CA_H */
