// C ABI of the library (declared in include/pink_b200.h): context state that
// stands for the device members of the reference's Trainer<...,true> and
// Mapper<...,true> objects (src/SelfOrganizingMapLib/Trainer.h:311-333,
// Mapper.h:210-229), the per-image launch sequences, host<->device staging and,
// with several ranks, the exchange of the per-shard best matching unit and of
// the rotation sets (peer memory over NVLink; NCCL as fallback).
#include "../../include/pink_b200.h"
#include "kernels.cuh"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <unistd.h>
#include <nccl.h>
#include <new>
#include <string>
#include <vector>

using namespace pinkb;

namespace {

thread_local std::string g_error;

int fail(int code, const std::string& msg)
{
    g_error = msg;
    return code;
}

#define CU_TRY(expr)                                                                              \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess)                                                                    \
            return fail(PINK_B200_ECUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));     \
    } while (0)

// ---- NCCL, resolved at run time so that single-GPU users need no NCCL at all ----
struct NcclApi
{
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi& nccl()
{
    static NcclApi api;
    if (api.handle) return api;
    api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!api.handle) api.handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!api.handle) return api;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(api.handle, "ncclCommInitRank"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(api.handle, "ncclAllGather"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(api.handle, "ncclCommDestroy"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(api.handle, "ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.AllGather && api.CommDestroy && api.GetErrorString;
    return api;
}

#define LAUNCH_TRY(expr)                                                                          \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess)                                                                    \
            return fail(PINK_B200_ECUDA, std::string("kernel launch failed in " #expr ": ") + cudaGetErrorString(e_)); \
    } while (0)

#define NCCL_TRY(expr)                                                                            \
    do {                                                                                          \
        ncclResult_t r_ = (expr);                                                                 \
        if (r_ != ncclSuccess)                                                                    \
            return fail(PINK_B200_ENCCL, std::string(#expr) + ": " + nccl().GetErrorString(r_)); \
    } while (0)

uint32_t round_up(uint32_t v, uint32_t m) { return (v + m - 1) / m * m; }

// Validation messages follow the reference's exceptions where it has one.
int make_geometry(const pink_b200_config& c, Geometry* g)
{
    if (c.n_neurons == 0 || c.channels == 0 || c.image_dim == 0 || c.neuron_dim == 0)
        return fail(PINK_B200_EINVAL, "SOM, image and neuron dimensions must be positive");
    if (c.n_rotations == 0 || (c.n_rotations != 1 && c.n_rotations % 4 != 0))
        return fail(PINK_B200_EINVAL, "Number of rotations must be 1 or larger then 1 and divisible by 4");
    if (c.ed_dim == 0) return fail(PINK_B200_EINVAL, "euclidean_distance_dim not defined");
    if (c.ed_dim > c.neuron_dim)
        return fail(PINK_B200_EINVAL, "Euclidean distance dimension larger than neuron dimension");
    if (c.interpolation != PINK_B200_BILINEAR)
        return fail(PINK_B200_EINVAL, "generate_rotated_images: unknown interpolation type");
    if (c.ed_shape != PINK_B200_QUADRATIC && c.ed_shape != PINK_B200_CIRCULAR)
        return fail(PINK_B200_EINVAL, "Unknown euclidean_distance_shape");
    if (c.dist_type > PINK_B200_UINT8) return fail(PINK_B200_EINVAL, "Unknown euclidean_distance_type");

    g->C = c.channels; g->id = c.image_dim; g->nd = c.neuron_dim; g->ed = c.ed_dim;
    g->R = c.n_rotations; g->flip = c.use_flip ? 1 : 0;
    g->T = g->R * (g->flip ? 2 : 1);
    g->q = g->R == 1 ? 0 : g->R / 4;
    g->off = static_cast<uint32_t>((g->nd - g->ed) * 0.5);
    const uint64_t P = (uint64_t)g->C * g->nd * g->nd, K = (uint64_t)g->C * g->ed * g->ed;
    if (P > (1u << 30)) return fail(PINK_B200_EINVAL, "neuron size too large");
    g->P = (uint32_t)P; g->Pp = round_up(g->P, 4);
    g->K = (uint32_t)K;
    g->mode = (int)c.dist_type;
    g->circle = nullptr;             // a context with a circular region uploads the table and sets this
    g->Kp = g->mode == kModeF32 ? round_up(g->K, 32) : round_up(g->K, 128);   // float: one 128-byte slice of the filter's TF32 planes
    // s32 accumulators: K * 255^2 (uint8) and 2 * K * 255^2 (uint16 cross term) must stay below 2^31.
    if (g->mode == kModeU8 && g->K > 33025) return fail(PINK_B200_EINVAL, "uint8 distance supports at most 33025 elements");
    if (g->mode == kModeU16 && g->K > 16512) return fail(PINK_B200_EINVAL, "uint16 distance supports at most 16512 elements");
    if (g->mode == kModeU16 && g->T > 65536) return fail(PINK_B200_EINVAL, "uint16 distance supports at most 65536 transforms");
    if ((uint64_t)g->T * g->R >= (1ull << 32)) return fail(PINK_B200_EINVAL, "too many rotations");
    return PINK_B200_OK;
}

size_t operand_plane_bytes(const Geometry& g, size_t rows)
{
    return rows * g.Kp * (g.mode == kModeF32 ? 4 : 1);
}

size_t norm_bytes(const Geometry& g, size_t rows)
{
    return rows * (g.mode == kModeU16 ? 8 : 4);
}

// Column span of every row of a circular distance region, restating the reference's CPU functor
// (src/ImageProcessingLib/circular_euclidean_distance.h:44-57): with center = nd / 2 and radius = ed / 2
// (integer divisions), region row i covers the neuron columns round(center - delta) .. round(center + delta) - 1,
// delta = sqrt(2 * radius * (i + 0.5) - (i + 0.5)^2) in double.  Returned in region-local columns
// (neuron column - offset); rows whose radicand is negative (odd ed) are empty.  False when a span leaves
// the ed x ed square the operands hold.
bool circle_table(uint32_t nd, uint32_t ed, std::vector<ushort2>* out)
{
    const uint32_t center = nd / 2, radius = ed / 2, off = static_cast<uint32_t>((nd - ed) * 0.5);
    out->assign(ed, make_ushort2(0, 0));
    for (uint32_t i = 0; i < ed; ++i) {
        const double arg = 2 * radius * (i + 0.5) - std::pow((i + 0.5), 2);
        if (!(arg >= 0.0)) continue;
        const double delta = std::sqrt(arg);
        const double lo = std::round(center - delta), hi = std::round(center + delta);
        if (!(hi > lo)) continue;
        if (lo < off || hi > off + ed) return false;
        (*out)[i] = make_ushort2((unsigned short)(lo - off), (unsigned short)(hi - off));
    }
    return true;
}

template <typename T>
void free_dev(T*& p)
{
    if (p) cudaFree(p);
    p = nullptr;
}

} // namespace

namespace pinkb {
// Geometry for the single-stage entries, which keep no device table of a circular region.
int geometry_from_config(const pink_b200_config* cfg, Geometry* g)
{
    if (!cfg || !g) return fail(PINK_B200_EINVAL, "null argument");
    if (cfg->ed_shape == PINK_B200_CIRCULAR)
        return fail(PINK_B200_EINVAL, "the single-stage entries support only the quadratic euclidean distance shape");
    return make_geometry(*cfg, g);
}
int report_error(int code, const char* msg) { return fail(code, msg); }
} // namespace pinkb

struct pink_b200_ctx
{
    pink_b200_config cfg{};
    Geometry g{};
    uint32_t first = 0, count = 0, stride = 1;    // local neuron j is global neuron first + j * stride
    uint32_t train_batch = 0, map_batch = 0;
    cudaStream_t stream = nullptr, copy_stream = nullptr, rot_stream = nullptr;
    cudaEvent_t copied[2] = { nullptr, nullptr }, consumed[2] = { nullptr, nullptr };
    // Training computes the rotation sets of kRotBatch images at once (they do not
    // depend on the SOM) into one of two alternating slots of transform buffers;
    // rot_stream is the training stream itself unless PINK_B200_ROT_OVERLAP is set.
    cudaEvent_t rotated[2] = { nullptr, nullptr }, rot_free[2] = { nullptr, nullptr };
    uint64_t rot_seq = 0;

    float* d_som = nullptr;
    void *d_a0 = nullptr, *d_a1 = nullptr, *d_anorm = nullptr;
    float *d_cs = nullptr, *d_sn = nullptr;
    float* d_factors = nullptr;       // this shard's columns of an N x N factor table, or ...
    short4* d_coords = nullptr; float* d_lut = nullptr;   // ... grid positions of all neurons + one factor per distance class
    FactorSource factor_source{};
    float* d_base = nullptr;   size_t base_imgs = 0;
    void *d_b0 = nullptr, *d_b1 = nullptr, *d_bnorm = nullptr; size_t b_imgs = 0;
    unsigned long long* d_keys = nullptr; size_t key_imgs = 0;
    BmuPair* d_pairs = nullptr;
    UpdateItem* d_items = nullptr; uint32_t* d_nitems = nullptr;   // per-step work list of the update
    // records of the ranks' best matching units exchanged by peer stores (world_size > 1, all ranks on one node)
    XchgRecord* d_xchg = nullptr; XchgRecord* xchg_peer[kXchgMaxRanks] = {}; bool xchg_on = false; unsigned long long xchg_seq = 0;
    bool peer_in_process[kXchgMaxRanks] = {};   // rank r lives in this process: its buffers are reached by plain peer access
    // value ranges for leaving out neurons that cannot change: per neuron {min |w|, max |w|}, per buffered image max |pixel|
    uint2* d_wrange = nullptr; uint32_t* d_rmax = nullptr;
    ushort2* d_circle = nullptr;      // column spans of a circular distance region (null: quadratic)
    // Rotation sets computed in shares (world_size > 1 with peer memory): every rank rotates its part of a
    // batch of images and copies the results into all ranks' transform buffers, which hold three batches.
    bool rot_shared = false;
    uint32_t share_group = 0;                              // ranks that share one batch's rotation work (consecutive ranks)
    cudaStream_t bcast_stream = nullptr, peer_stream[kXchgMaxRanks] = {};   // one copy stream per destination rank, joined on bcast_stream
    cudaEvent_t share_rotated = nullptr, bcast_done[3] = { nullptr, nullptr, nullptr }, peer_sent[kXchgMaxRanks] = {};
    unsigned long long* d_rotflag = nullptr;               // [3 batches][world]: batch number + 1 of the share that arrived
    unsigned long long* peer_rotflag[kXchgMaxRanks] = {};
    float* peer_base[kXchgMaxRanks] = {};
    uint8_t* peer_b0[kXchgMaxRanks] = {}; uint8_t* peer_b1[kXchgMaxRanks] = {}; uint8_t* peer_bnorm[kXchgMaxRanks] = {};
    uint32_t* peer_rmax[kXchgMaxRanks] = {};
    uint64_t share_seq = 0;                                // batches handled so far (all ranks count alike)
    unsigned long long* d_stats = nullptr;   // [0] neurons with a non-zero factor, [1] neurons written back, summed over steps
    uint64_t launches = 0;            // kernels launched by this context so far
    bool fuse_update = false;         // the update kernel finds the best matching unit and its work list itself
    // Whole batches of training steps in one persistent kernel (train_steps.cu) where the geometry allows it.
    bool plan_ok = false;             // the persistent kernel can run this geometry
    bool use_steps = false;           // ... and this context uses it (decided when training starts)
    StepPlan plan{};
    uint32_t* d_owners = nullptr;     // [plan.grid][plan.owned_per_block]: which block rewrites which neuron
    StepCtrl* d_ctrl = nullptr;
    unsigned long long* d_stamps = nullptr; size_t stamps_cap = 0;   // opt-in device-timer stamps, 8 per profiled step
    std::vector<cudaEvent_t> prof_launch_events; size_t prof_launches = 0, prof_launch_images = 0;
    // switches (pink_b200_set_option)
    int opt_step_kernel = 0;          // 0 persistent kernel where possible, 1 two kernels per image, 2 split update path
    int opt_exchange = 0;             // 0 peer memory where possible, 1 NCCL all-gather
    int opt_rotation_sharing = -1;    // -1 pairs of ranks, 0 every rank rotates everything, g >= 2 groups of g ranks
    int opt_mma_pairs = 1;
    int opt_cooperative = 1;          // 0: persistent kernel launched without the cooperative attribute
    int opt_f32_filter = 1;           // float32 mapping: tensor-core estimate + exact pass where the geometry allows it
    // float32 mapping filter: TF32 word planes and float norms of the SOM operand (valid while the SOM is unchanged)
    // and of one mapping batch of transforms, the estimate matrix and the pass's counters
    float* d_af_hi = nullptr; float* d_af_lo = nullptr; float* d_af_norm = nullptr; bool af_valid = false;
    float* d_bf_hi = nullptr; float* d_bf_lo = nullptr; float* d_bf_norm = nullptr; float* d_est = nullptr; size_t filter_imgs = 0;
    unsigned long long* d_filter_stats = nullptr;     // {exact evaluations, bits of the largest estimate error seen}
    unsigned long long filter_pairs = 0;              // (neuron, transform) pairs estimated so far
    long long opt_exchange_timeout_ms = 20000;
    bool failed = false;              // a device-side wait expired: the map may be inconsistent, training is refused
    uint32_t* d_counts = nullptr;
    uint32_t* d_bmu_log = nullptr; size_t bmu_log_cap = 0, bmu_log_n = 0;
    int* d_status = nullptr;
    float* d_images[2] = { nullptr, nullptr }; size_t image_cap = 0;
    float* d_dist = nullptr; uint32_t* d_rot = nullptr; size_t out_imgs = 0;
    bool have_som = false, have_factors = false;
    ncclComm_t comm = nullptr;
    // opt-in phase timing: four events per profiled training step, two per rotation batch
    std::vector<cudaEvent_t> prof_events, prof_rot_events;
    size_t prof_cap = 0, prof_used = 0, prof_rot_used = 0;

    size_t image_size() const { return (size_t)g.C * g.id * g.id; }
};

namespace {

// A base rotation is staged in shared memory when it fits; only then can the
// float copy in global memory be skipped (mapping never reads it back).
bool base_fits_smem(const Geometry& g) { return (size_t)g.P * sizeof(float) <= 200 * 1024; }

int ensure_transform_buffers(pink_b200_ctx* c, size_t imgs, size_t base_needed)
{
    const Geometry& g = c->g;
    if (c->b_imgs < imgs) {
        free_dev(c->d_b0); free_dev(c->d_b1); free_dev(c->d_bnorm);
        const size_t rows = imgs * g.T;
        CU_TRY(cudaMalloc(&c->d_b0, operand_plane_bytes(g, rows)));
        CU_TRY(cudaMemsetAsync(c->d_b0, 0, operand_plane_bytes(g, rows), c->stream));
        if (g.mode == kModeU16) {
            CU_TRY(cudaMalloc(&c->d_b1, operand_plane_bytes(g, rows)));
            CU_TRY(cudaMemsetAsync(c->d_b1, 0, operand_plane_bytes(g, rows), c->stream));
        }
        CU_TRY(cudaMalloc(&c->d_bnorm, norm_bytes(g, rows)));
        c->b_imgs = imgs;
    }
    if (c->base_imgs < base_needed) {
        free_dev(c->d_base);
        CU_TRY(cudaMalloc(&c->d_base, base_needed * (g.q ? g.q : 1) * (size_t)g.P * sizeof(float)));
        c->base_imgs = base_needed;
    }
    const size_t key_imgs_needed = imgs;
    if (c->key_imgs < key_imgs_needed) {
        free_dev(c->d_keys);
        CU_TRY(cudaMalloc(&c->d_keys, imgs * c->count * sizeof(unsigned long long)));
        LAUNCH_TRY(launch_fill_keys(c->d_keys, imgs * c->count, c->stream));
        c->launches += 1;
        c->key_imgs = imgs;
    }
    CU_TRY(cudaStreamSynchronize(c->stream));   // initialisation complete before other streams touch the buffers
    return PINK_B200_OK;
}

int ensure_image_staging(pink_b200_ctx* c, size_t imgs)
{
    if (c->image_cap >= imgs) return PINK_B200_OK;
    for (int i = 0; i < 2; ++i) {
        free_dev(c->d_images[i]);
        CU_TRY(cudaMalloc(&c->d_images[i], imgs * c->image_size() * sizeof(float)));
    }
    c->image_cap = imgs;
    return PINK_B200_OK;
}

int check_status(pink_b200_ctx* c)
{
    int st = 0;
    CU_TRY(cudaMemcpyAsync(&st, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    if (st != kDevOk) {
        // Sticky: the steps after the expired wait ran on whatever state it left, and with several ranks
        // the exchange counters no longer agree.  The context only answers get_som / destroy from here on.
        c->failed = true;
        return fail(PINK_B200_ETIMEOUT, "a bounded device-side wait expired (code " + std::to_string(st) + ")");
    }
    return PINK_B200_OK;
}

constexpr uint32_t kRotBatch = kStepBatchMax;

// float32 distances through the tensor-core estimate + exact pass: possible when the exact pass's candidate lists
// fit shared memory (T) and the operand rows are whole 128-byte slices
bool uses_filter(const pink_b200_ctx* c)
{
    return c->g.mode == kModeF32 && c->opt_f32_filter && c->g.Kp % 32 == 0 && c->g.T <= 12800;
}

// Bound of the estimate's error relative to |a|^2 + |b|^2 (derived in filter_f32.cu): 3 * K / 16 * 2^-23 + 2^-17
float filter_eps(uint32_t K) { return (float)(3.0 * K / 16.0 * 1.1920928955078125e-7 + 7.62939453125e-6); }

int ensure_filter_buffers(pink_b200_ctx* c, size_t imgs)
{
    const Geometry& g = c->g;
    if (!c->d_af_hi) {
        const size_t elems = (size_t)c->count * g.Kp;
        CU_TRY(cudaMalloc(&c->d_af_hi, elems * sizeof(float)));
        CU_TRY(cudaMalloc(&c->d_af_lo, elems * sizeof(float)));
        CU_TRY(cudaMalloc(&c->d_af_norm, (size_t)c->count * sizeof(float)));
        CU_TRY(cudaMalloc(&c->d_filter_stats, 2 * sizeof(unsigned long long)));
        CU_TRY(cudaMemsetAsync(c->d_filter_stats, 0, 2 * sizeof(unsigned long long), c->stream));
        c->af_valid = false;
    }
    if (c->filter_imgs < imgs) {
        free_dev(c->d_bf_hi); free_dev(c->d_bf_lo); free_dev(c->d_bf_norm); free_dev(c->d_est);
        const size_t rows = imgs * g.T;
        CU_TRY(cudaMalloc(&c->d_bf_hi, rows * g.Kp * sizeof(float)));
        CU_TRY(cudaMalloc(&c->d_bf_lo, rows * g.Kp * sizeof(float)));
        // the rotation kernel writes K values per row; the padding up to Kp stays zero
        CU_TRY(cudaMemsetAsync(c->d_bf_hi, 0, rows * g.Kp * sizeof(float), c->stream));
        CU_TRY(cudaMemsetAsync(c->d_bf_lo, 0, rows * g.Kp * sizeof(float), c->stream));
        CU_TRY(cudaMalloc(&c->d_bf_norm, rows * sizeof(float)));
        CU_TRY(cudaMalloc(&c->d_est, rows * c->count * sizeof(float)));
        c->filter_imgs = imgs;
    }
    return PINK_B200_OK;
}

// One training step on image `slot_img` of the transform buffers (its rotation
// set is already there): distance + minimum over transforms, best matching
// unit (+ exchange between ranks), neighbourhood update.
int train_step(pink_b200_ctx* c, size_t slot_img, uint32_t* bmu_slot)
{
    const Geometry& g = c->g;
    const size_t esz = g.mode == kModeF32 ? 4 : 1;
    const size_t row0 = slot_img * g.T;
    cudaEvent_t* ev = nullptr;
    if (c->prof_used < c->prof_cap) ev = &c->prof_events[4 * c->prof_used++];
    DistanceArgs da{};
    da.a0 = c->d_a0; da.a1 = c->d_a1; da.anorm = c->d_anorm; da.n = c->count;
    da.b0 = static_cast<uint8_t*>(c->d_b0) + row0 * g.Kp * esz;
    da.b1 = c->d_b1 ? static_cast<uint8_t*>(c->d_b1) + row0 * g.Kp * esz : nullptr;
    da.bnorm = static_cast<uint8_t*>(c->d_bnorm) + row0 * (g.mode == kModeU16 ? 8 : 4);
    da.n_img = 1;
    da.keys = c->d_keys; da.s_out = nullptr; da.status = c->d_status; da.single_cta = !c->opt_mma_pairs;
    BmuArgs ba{};
    ba.keys = c->d_keys; ba.n = c->count; ba.first_neuron = c->first; ba.neuron_stride = c->stride; ba.shift = key_shift(g.mode);
    ba.pairs = c->d_pairs; ba.rank = c->cfg.rank; ba.world = c->cfg.world_size;
    ba.factors = c->factor_source; ba.items = c->d_items; ba.n_items = c->d_nitems;
    ba.counts = c->d_counts; ba.bmu_log = bmu_slot;
    ba.R = g.R; ba.q = g.q; ba.nd = g.nd;
    ba.magic_R = g.R == 1 ? 0u : (uint32_t)((1ull << 32) / g.R) + 1;
    ba.magic_q = g.q <= 1 ? 0u : (uint32_t)((1ull << 32) / g.q) + 1;
    ba.arrive = c->d_nitems + 1;
    ba.stats = c->d_stats;
    ba.status = c->d_status;
    ba.xchg_timeout_ns = (unsigned long long)std::max<long long>(1, c->opt_exchange_timeout_ms) * 1000000ull;
    // Fused form: the update kernel reduces the keys (or the exchanged records) and derives its
    // work list itself; otherwise a reduction and a compaction kernel run in between.
    const bool fused = c->fuse_update;
    const bool multi = c->cfg.world_size > 1;
    const bool peer = multi && fused && c->xchg_on;
    if (peer) {
        // this rank's record goes into every rank's array by peer stores; the update kernel waits for all
        ba.xchg_seq = ++c->xchg_seq;
        ba.xchg_local = c->d_xchg;
        for (uint32_t r = 0; r < c->cfg.world_size; ++r) ba.xchg_peer[r] = c->xchg_peer[r];
    }
    // with several ranks the distance kernel's last block reduces the shard's keys to its record
    const bool tail = multi && distance_has_tail(g);
    if (tail) { da.tail = &ba; da.tail_counter = c->d_nitems + 2; }
    const char* why = "";
    if (ev) CU_TRY(cudaEventRecord(ev[0], c->stream));
    cudaError_t e = cudaSuccess;
    if (uses_filter(c)) {
        // float32: estimate of every pair on the tensor cores, exact sums for the transforms it cannot rule out.
        // The update rewrites operand rows, so the SOM's planes are rebuilt for every image.
        const float* A = static_cast<const float*>(c->d_a0);
        const float* B = static_cast<const float*>(c->d_b0) + row0 * g.Kp;
        LAUNCH_TRY(launch_split_tf32(A, c->count, g.Kp, c->d_af_hi, c->d_af_lo, c->d_af_norm, c->stream));
        LAUNCH_TRY(launch_split_tf32(B, g.T, g.Kp, c->d_bf_hi, c->d_bf_lo, c->d_bf_norm, c->stream));
        DistanceArgs fa = da;
        fa.a0 = c->d_af_hi; fa.a1 = c->d_af_lo; fa.anorm = c->d_af_norm;
        fa.b0 = c->d_bf_hi; fa.b1 = c->d_bf_lo; fa.bnorm = c->d_bf_norm;
        fa.s_out = c->d_est;
        e = launch_distance_tf32(g, fa, c->stream, &why);
        if (e == cudaSuccess) {
            why = "refine_f32_kernel launch";
            e = launch_refine_f32(g, A, c->d_af_norm, c->count, B, c->d_bf_norm, 1, c->d_est, filter_eps(g.K), c->d_keys,
                                  c->d_filter_stats, c->stream);
        }
        c->filter_pairs += (unsigned long long)c->count * g.T;
        c->launches += 3;
    } else {
        e = launch_distance(g, da, c->stream, &why);
    }
    if (e != cudaSuccess) return fail(PINK_B200_ECUDA, std::string(why) + ": " + cudaGetErrorString(e));
    if (ev) CU_TRY(cudaEventRecord(ev[1], c->stream));
    if (!multi) {
        if (!fused) { LAUNCH_TRY(launch_bmu(ba, 3, c->stream)); c->launches += 2; }
    } else {
        if (!tail) { LAUNCH_TRY(launch_bmu(ba, 1, c->stream)); c->launches += 1; }
        if (!peer) NCCL_TRY(nccl().AllGather(c->d_pairs + c->cfg.rank, c->d_pairs, 2, ncclUint64, c->comm, c->stream));
        if (!fused) { LAUNCH_TRY(launch_bmu(ba, 2, c->stream)); c->launches += 1; }
    }
    UpdateArgs ua{};
    ua.som = c->d_som;
    ua.base = c->d_base + slot_img * (g.q ? g.q : 1) * (size_t)g.P;
    ua.items = c->d_items; ua.n_items = c->d_nitems; ua.n = c->count;
    ua.a0 = c->d_a0; ua.a1 = c->d_a1; ua.anorm = c->d_anorm;
    ua.wrange = fused ? c->d_wrange : nullptr;
    ua.rmax = fused && c->d_wrange ? c->d_rmax + slot_img : nullptr;
    if (ev) CU_TRY(cudaEventRecord(ev[2], c->stream));
    if (fused) LAUNCH_TRY(launch_update_fused(g, ua, ba, c->stream, c->d_status));
    else LAUNCH_TRY(launch_update(g, ua, c->stream, c->d_status));
    c->launches += 2;                 // distance + update
    if (ev) CU_TRY(cudaEventRecord(ev[3], c->stream));
    return PINK_B200_OK;
}

// cnt (<= kRotBatch) consecutive training steps on the images whose rotation sets start at image `slot_img`
// of the transform buffers, in one launch of the persistent kernel.
int train_steps_batch(pink_b200_ctx* c, size_t slot_img, uint32_t cnt, uint32_t* bmu_slots)
{
    const Geometry& g = c->g;
    StepArgs a{};
    a.a0 = c->d_a0; a.a1 = c->d_a1; a.anorm = c->d_anorm; a.n = c->count;
    a.b0 = c->d_b0; a.b1 = c->d_b1; a.bnorm = c->d_bnorm;
    a.b_rows = (uint32_t)(c->b_imgs * g.T);
    a.b_row0 = (uint32_t)(slot_img * g.T);
    a.keys = c->d_keys;
    a.som = c->d_som;
    a.base = c->d_base + slot_img * (g.q ? g.q : 1) * (size_t)g.P;
    a.wrange = c->d_wrange;
    a.rmax = c->d_wrange ? c->d_rmax + slot_img : nullptr;
    a.factors = c->factor_source;
    a.owners = c->d_owners;
    a.n_img = cnt; a.first_neuron = c->first; a.neuron_stride = c->stride; a.rank = c->cfg.rank; a.world = c->cfg.world_size;
    a.counts = c->d_counts; a.bmu_log = bmu_slots; a.stats = c->d_stats; a.status = c->d_status;
    a.ctrl = c->d_ctrl;
    a.stamps = nullptr;
    a.plain_launch = c->opt_cooperative ? 0u : 1u;
    if (c->cfg.world_size > 1) {
        a.xchg_local = c->d_xchg;
        for (uint32_t r = 0; r < c->cfg.world_size; ++r) a.xchg_peer[r] = c->xchg_peer[r];
        a.xchg_seq0 = c->xchg_seq + 1;
        c->xchg_seq += cnt;
    }
    a.xchg_timeout_ns = (unsigned long long)std::max<long long>(1, c->opt_exchange_timeout_ms) * 1000000ull;
    cudaEvent_t* ev = nullptr;
    if (c->prof_used < c->prof_cap) {
        if (c->d_stamps && c->prof_used + cnt <= c->stamps_cap) a.stamps = c->d_stamps + (size_t)kStepStampWords * c->plan.grid * c->prof_used;
        if (2 * (c->prof_launches + 1) <= c->prof_launch_events.size()) ev = &c->prof_launch_events[2 * c->prof_launches];
        c->prof_used += std::min<size_t>(cnt, c->prof_cap - c->prof_used);
    }
    CU_TRY(cudaMemsetAsync(c->d_ctrl, 0xFF, sizeof(StepCtrl), c->stream));
    if (ev) CU_TRY(cudaEventRecord(ev[0], c->stream));
    const char* why = "";
    cudaError_t e = launch_train_steps(g, c->plan, a, c->stream, &why);
    if (e != cudaSuccess) return fail(PINK_B200_ECUDA, std::string(why) + ": " + cudaGetErrorString(e));
    if (ev) { CU_TRY(cudaEventRecord(ev[1], c->stream)); c->prof_launches += 1; c->prof_launch_images += cnt; }
    c->launches += 1;
    return PINK_B200_OK;
}

// m sequential steps over images resident on the device.  `ready` (nullable) is
// an event the rotation stream must wait for before reading the images.
static int train_chunk_shared(pink_b200_ctx* c, const float* d_images, uint64_t m, uint32_t* log, cudaEvent_t ready);

int train_chunk(pink_b200_ctx* c, const float* d_images, uint64_t m, uint32_t* log, cudaEvent_t ready)
{
    if (m == 0) return PINK_B200_OK;
    if (c->rot_shared) return train_chunk_shared(c, d_images, m, log, ready);
    const Geometry& g = c->g;
    const size_t esz = g.mode == kModeF32 ? 4 : 1, isz = c->image_size();
    for (uint64_t s0 = 0; s0 < m; s0 += kRotBatch) {
        const uint32_t cnt = (uint32_t)(m - s0 < kRotBatch ? m - s0 : kRotBatch);
        const size_t slot = (size_t)(c->rot_seq++ & 1) * kRotBatch;
        const size_t row0 = slot * g.T;
        CU_TRY(cudaStreamWaitEvent(c->rot_stream, c->rot_free[slot ? 1 : 0], 0));
        if (ready && s0 == 0) CU_TRY(cudaStreamWaitEvent(c->rot_stream, ready, 0));
        cudaEvent_t* ev = nullptr;
        if (c->prof_used < c->prof_cap && 2 * (c->prof_rot_used + 1) <= c->prof_rot_events.size())
            ev = &c->prof_rot_events[2 * c->prof_rot_used++];
        if (ev) CU_TRY(cudaEventRecord(ev[0], c->rot_stream));
        CU_TRY(cudaMemsetAsync(c->d_rmax + slot, 0, cnt * sizeof(uint32_t), c->rot_stream));
        LAUNCH_TRY(launch_rotate(g, d_images + s0 * isz, cnt, c->d_cs, c->d_sn,
                                 c->d_base + slot * (g.q ? g.q : 1) * (size_t)g.P,
                                 static_cast<uint8_t*>(c->d_b0) + row0 * g.Kp * esz,
                                 c->d_b1 ? static_cast<uint8_t*>(c->d_b1) + row0 * g.Kp * esz : nullptr,
                                 static_cast<uint8_t*>(c->d_bnorm) + row0 * (g.mode == kModeU16 ? 8 : 4),
                                 c->rot_stream, c->d_rmax + slot));
        c->launches += 1;
        if (ev) CU_TRY(cudaEventRecord(ev[1], c->rot_stream));
        CU_TRY(cudaEventRecord(c->rotated[slot ? 1 : 0], c->rot_stream));
        CU_TRY(cudaStreamWaitEvent(c->stream, c->rotated[slot ? 1 : 0], 0));
        if (c->use_steps) {
            int rc = train_steps_batch(c, slot, cnt, log + s0);
            if (rc) return rc;
        } else {
            for (uint32_t i = 0; i < cnt; ++i) {
                int rc = train_step(c, slot + i, log + s0 + i);
                if (rc) return rc;
            }
        }
        CU_TRY(cudaEventRecord(c->rot_free[slot ? 1 : 0], c->stream));
    }
    return PINK_B200_OK;
}

// The same over several ranks that share the rotation work (rot_shared): of every batch of kRotBatch images
// a rank rotates a contiguous part, copies the results (base rotations, operand rows, norms, pixel maximum)
// into every other rank's transform buffers on a copy stream, and then raises its flag in every rank's
// flag row; a rank starts the steps of a batch when all flags of the batch are up.  The part of batch b + 1
// is rotated before the steps of batch b, so that its copies travel while those steps run.  The buffers hold
// three batches: the ranks are at most one step apart (they exchange a record every step), so a batch two
// ahead never lands in memory a slower rank still reads.
static int train_chunk_shared(pink_b200_ctx* c, const float* d_images, uint64_t m, uint32_t* log, cudaEvent_t ready)
{
    const Geometry& g = c->g;
    const uint32_t W = c->cfg.world_size, rank = c->cfg.rank;
    // the ranks sharing with this one: [g0, g0 + G), this rank the gr-th of them
    const uint32_t g0 = rank / c->share_group * c->share_group, G = std::min(c->share_group, W - g0), gr = rank - g0;
    const size_t esz = g.mode == kModeF32 ? 4 : 1, isz = c->image_size(), nbase = g.q ? g.q : 1;
    const size_t base_img = nbase * (size_t)g.P * sizeof(float), op_img = (size_t)g.T * g.Kp * esz;
    const size_t norm_img = (size_t)g.T * (g.mode == kModeU16 ? 8 : 4);
    if (ready) CU_TRY(cudaStreamWaitEvent(c->stream, ready, 0));
    const uint64_t batches = (m + kRotBatch - 1) / kRotBatch;
    auto produce = [&](uint64_t b) -> int {
        const uint64_t seq = c->share_seq + b;
        const uint32_t ring = (uint32_t)(seq % 3);
        const size_t slot = (size_t)ring * kRotBatch;
        const uint32_t cnt = (uint32_t)std::min<uint64_t>(kRotBatch, m - b * kRotBatch);
        const uint32_t per = (cnt + G - 1) / G, lo = std::min(gr * per, cnt), hi = std::min(lo + per, cnt);
        // the copies that last read this part of the buffers (three batches ago) are over
        CU_TRY(cudaStreamWaitEvent(c->stream, c->bcast_done[ring], 0));
        if (hi > lo) {
            CU_TRY(cudaMemsetAsync(c->d_rmax + slot + lo, 0, (hi - lo) * sizeof(uint32_t), c->stream));
            const size_t row0 = (slot + lo) * g.T;
            cudaEvent_t* ev = nullptr;
            if (c->prof_used < c->prof_cap && 2 * (c->prof_rot_used + 1) <= c->prof_rot_events.size())
                ev = &c->prof_rot_events[2 * c->prof_rot_used++];
            if (ev) CU_TRY(cudaEventRecord(ev[0], c->stream));
            LAUNCH_TRY(launch_rotate(g, d_images + (b * kRotBatch + lo) * isz, hi - lo, c->d_cs, c->d_sn,
                                     c->d_base + (slot + lo) * nbase * (size_t)g.P,
                                     static_cast<uint8_t*>(c->d_b0) + row0 * g.Kp * esz,
                                     c->d_b1 ? static_cast<uint8_t*>(c->d_b1) + row0 * g.Kp * esz : nullptr,
                                     static_cast<uint8_t*>(c->d_bnorm) + row0 * (g.mode == kModeU16 ? 8 : 4),
                                     c->stream, c->d_rmax + slot + lo));
            c->launches += 1;
            if (ev) CU_TRY(cudaEventRecord(ev[1], c->stream));
        }
        // one stream per destination, so that the copies to different ranks use different copy engines and
        // links at the same time; a destination's flag follows its copies in its stream
        CU_TRY(cudaEventRecord(c->share_rotated, c->stream));
        for (uint32_t p = g0; p < g0 + G; ++p) {
            if (p == rank) continue;
            cudaStream_t ps = c->peer_stream[p];
            CU_TRY(cudaStreamWaitEvent(ps, c->share_rotated, 0));
            if (hi > lo) {
                const size_t first = slot + lo, n = hi - lo;
                CU_TRY(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(c->peer_base[p]) + first * base_img,
                                       reinterpret_cast<uint8_t*>(c->d_base) + first * base_img, n * base_img, cudaMemcpyDefault, ps));
                CU_TRY(cudaMemcpyAsync(c->peer_b0[p] + first * op_img, static_cast<uint8_t*>(c->d_b0) + first * op_img, n * op_img,
                                       cudaMemcpyDefault, ps));
                if (c->d_b1)
                    CU_TRY(cudaMemcpyAsync(c->peer_b1[p] + first * op_img, static_cast<uint8_t*>(c->d_b1) + first * op_img, n * op_img,
                                           cudaMemcpyDefault, ps));
                CU_TRY(cudaMemcpyAsync(c->peer_bnorm[p] + first * norm_img, static_cast<uint8_t*>(c->d_bnorm) + first * norm_img,
                                       n * norm_img, cudaMemcpyDefault, ps));
                CU_TRY(cudaMemcpyAsync(c->peer_rmax[p] + first, c->d_rmax + first, n * sizeof(uint32_t), cudaMemcpyDefault, ps));
            }
            LAUNCH_TRY(launch_flag_publish(&c->peer_rotflag[p], 1, ring * W + rank, seq + 1, ps));
            c->launches += 1;
            CU_TRY(cudaEventRecord(c->peer_sent[p], ps));
            CU_TRY(cudaStreamWaitEvent(c->bcast_stream, c->peer_sent[p], 0));
        }
        CU_TRY(cudaEventRecord(c->bcast_done[ring], c->bcast_stream));
        return PINK_B200_OK;
    };
    int rc = produce(0);
    if (rc) return rc;
    for (uint64_t b = 0; b < batches; ++b) {
        if (b + 1 < batches) { rc = produce(b + 1); if (rc) return rc; }
        const uint64_t seq = c->share_seq + b;
        const uint32_t ring = (uint32_t)(seq % 3);
        const uint32_t cnt = (uint32_t)std::min<uint64_t>(kRotBatch, m - b * kRotBatch);
        // This rank's own share of the batch must have left (copies and flag) before its steps begin: the
        // update kernel fills every SM while it waits for the other ranks' records, and they wait for this
        // flag -- whose kernel could then find no SM to run on.
        CU_TRY(cudaStreamWaitEvent(c->stream, c->bcast_done[ring], 0));
        LAUNCH_TRY(launch_flag_wait(c->d_rotflag + ring * W + g0, G, gr, seq + 1, c->d_status,
                                    (unsigned long long)std::max<long long>(1, c->opt_exchange_timeout_ms) * 1000000ull, c->stream));
        c->launches += 1;
        if (c->use_steps) {
            rc = train_steps_batch(c, (size_t)ring * kRotBatch, cnt, log + b * kRotBatch);
            if (rc) return rc;
        } else {
            for (uint32_t i = 0; i < cnt; ++i) {
                rc = train_step(c, (size_t)ring * kRotBatch + i, log + b * kRotBatch + i);
                if (rc) return rc;
            }
        }
    }
    c->share_seq += batches;
    return PINK_B200_OK;
}

void release_peer_exchange(pink_b200_ctx* c)
{
    for (uint32_t r = 0; r < kXchgMaxRanks; ++r) {
        if (c->xchg_peer[r] && c->xchg_peer[r] != c->d_xchg && !c->peer_in_process[r]) cudaIpcCloseMemHandle(c->xchg_peer[r]);
        c->xchg_peer[r] = nullptr;
    }
    if (c->d_xchg) cudaFree(c->d_xchg);
    c->d_xchg = nullptr;
    c->xchg_on = false;
    for (uint32_t r = 0; r < kXchgMaxRanks; ++r) {
        if (r != c->cfg.rank && !c->peer_in_process[r]) {
            if (c->peer_rotflag[r]) cudaIpcCloseMemHandle(c->peer_rotflag[r]);
            if (c->peer_base[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
            if (c->peer_b0[r]) cudaIpcCloseMemHandle(c->peer_b0[r]);
            if (c->peer_b1[r]) cudaIpcCloseMemHandle(c->peer_b1[r]);
            if (c->peer_bnorm[r]) cudaIpcCloseMemHandle(c->peer_bnorm[r]);
            if (c->peer_rmax[r]) cudaIpcCloseMemHandle(c->peer_rmax[r]);
        }
        c->peer_rotflag[r] = nullptr; c->peer_base[r] = nullptr; c->peer_b0[r] = nullptr; c->peer_b1[r] = nullptr;
        c->peer_bnorm[r] = nullptr; c->peer_rmax[r] = nullptr;
    }
    if (c->d_rotflag) cudaFree(c->d_rotflag);
    c->d_rotflag = nullptr;
    c->rot_shared = false;
}

// Sets up the exchange of best-matching-unit records through peer memory: every rank
// allocates its record array, the CUDA IPC handles travel once through an NCCL all-gather,
// and each rank maps the other ranks' arrays.  The exchange is switched on only if every
// rank could map every array and no two ranks share a GPU (a kernel that waits for a peer's
// record must never share its GPU with the kernel that writes it); otherwise the per-step
// NCCL all-gather stays in use.  Option "exchange" = 1 keeps NCCL too.
int setup_peer_exchange(pink_b200_ctx* c)
{
    const uint32_t W = c->cfg.world_size, rank = c->cfg.rank;
    // handles: 0 record ring; 1..6 the transform buffers and the flag rows of the shared rotation
    // (pid, device, ptr: ranks that live in one process -- a group driving several GPUs -- cannot open each other's
    //  IPC handles; they enable peer access and use the device pointers themselves)
    struct Hello { cudaIpcMemHandle_t handle[7]; void* ptr[7]; char bus[32]; long long pid; int device;
                   uint32_t want; uint32_t share; uint32_t ok; };
    Hello mine{};
    std::vector<Hello> all(W);
    Hello* d_all = nullptr;
    // (distance codes must leave room for the 8-bit tag of a record word: 65535^2 * K < 2^56)
    mine.want = W <= kXchgMaxRanks && (c->fuse_update || (c->plan_ok && c->opt_step_kernel == 0)) && c->g.K < (1u << 24)
                && c->opt_exchange == 0;
    mine.pid = (long long)getpid();
    mine.device = c->cfg.device;
    if (mine.want) {
        const size_t bytes = (size_t)kXchgSlots * W * sizeof(XchgRecord);
        CU_TRY(cudaMalloc(&c->d_xchg, bytes));
        CU_TRY(cudaMemsetAsync(c->d_xchg, 0, bytes, c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));          // zeroed before any rank can learn the handle
        mine.ptr[0] = c->d_xchg;
        if (cudaIpcGetMemHandle(&mine.handle[0], c->d_xchg) != cudaSuccess) { cudaGetLastError(); mine.want = 0; }
        if (cudaDeviceGetPCIBusId(mine.bus, sizeof(mine.bus), c->cfg.device) != cudaSuccess) { cudaGetLastError(); mine.want = 0; }
    }
    // Shared rotation: the transform buffers get their final size now (three training batches, or the mapping
    // batch if that is larger) because the other ranks map them.  By default pairs of consecutive ranks share:
    // measured on eight B200, pairs gain 7 % over every rank rotating everything (25.4 k against 23.8 k
    // images/s) and on two B200 6 %, while sharing among all eight loses (18.4 k): the copies to seven
    // destinations (164 MB per rank and batch in each direction) slow the other kernels down by more than the
    // rotation work they save.
    // Option "rotation_sharing" (pink_b200_set_option): g >= 2 makes groups of g consecutive ranks share,
    // 0 switches sharing off, -1 is this default.  `share` carries the group size.
    uint32_t group = 0;
    if (mine.want && c->opt_rotation_sharing != 0)
        group = c->opt_rotation_sharing >= 2 ? (uint32_t)std::min<long>(c->opt_rotation_sharing, W) : std::min<uint32_t>(W, 2);
    mine.share = group;
    if (mine.share) {
        const size_t imgs = std::max<size_t>(3 * kRotBatch, c->map_batch);
        int rc0 = ensure_transform_buffers(c, imgs, 3 * kRotBatch);
        if (rc0) return rc0;
        CU_TRY(cudaMalloc(&c->d_rotflag, 3 * W * sizeof(unsigned long long)));
        CU_TRY(cudaMemsetAsync(c->d_rotflag, 0, 3 * W * sizeof(unsigned long long), c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));
        void* bufs[6] = { c->d_base, c->d_b0, c->d_b1, c->d_bnorm, c->d_rmax, c->d_rotflag };
        for (int i = 0; i < 6; ++i) {
            mine.ptr[1 + i] = bufs[i];
            if (bufs[i] && cudaIpcGetMemHandle(&mine.handle[1 + i], bufs[i]) != cudaSuccess) { cudaGetLastError(); mine.share = 0; }
        }
    }
    CU_TRY(cudaMalloc(&d_all, W * sizeof(Hello)));
    auto gather = [&]() -> int {
        CU_TRY(cudaMemcpyAsync(d_all + rank, &mine, sizeof(Hello), cudaMemcpyHostToDevice, c->stream));
        NCCL_TRY(nccl().AllGather(d_all + rank, d_all, sizeof(Hello), ncclUint8, c->comm, c->stream));
        CU_TRY(cudaMemcpyAsync(all.data(), d_all, W * sizeof(Hello), cudaMemcpyDeviceToHost, c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));
        return PINK_B200_OK;
    };
    int rc = gather();
    if (rc) { cudaFree(d_all); return rc; }
    bool ok = true, share = true;
    for (uint32_t r = 0; r < W; ++r) {
        ok = ok && all[r].want;
        share = share && all[r].share == group && group >= 2;
        for (uint32_t q = 0; q < r; ++q) ok = ok && std::strncmp(all[r].bus, all[q].bus, sizeof(mine.bus)) != 0;
    }
    share = share && ok;
    auto open = [&](uint32_t r, int i, void** out) {
        if (all[r].pid == mine.pid) {
            // same process: direct peer access to the other rank's device
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, c->cfg.device, all[r].device) == cudaSuccess && can) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(all[r].device, 0);
                if (e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled) {
                    cudaGetLastError();
                    *out = all[r].ptr[i];
                    c->peer_in_process[r] = true;
                    return true;
                }
            }
            cudaGetLastError();
            *out = nullptr;
            return false;
        }
        if (cudaIpcOpenMemHandle(out, all[r].handle[i], cudaIpcMemLazyEnablePeerAccess) == cudaSuccess) return true;
        cudaGetLastError();
        *out = nullptr;
        return false;
    };
    if (ok) {
        for (uint32_t r = 0; r < W && ok; ++r) {
            if (r == rank) { c->xchg_peer[r] = c->d_xchg; continue; }
            void* ptr = nullptr;
            ok = open(r, 0, &ptr);
            c->xchg_peer[r] = static_cast<XchgRecord*>(ptr);
        }
    }
    if (share) {
        for (uint32_t r = 0; r < W && share; ++r) {
            if (r == rank) {
                c->peer_base[r] = c->d_base; c->peer_b0[r] = static_cast<uint8_t*>(c->d_b0);
                c->peer_b1[r] = static_cast<uint8_t*>(c->d_b1); c->peer_bnorm[r] = static_cast<uint8_t*>(c->d_bnorm);
                c->peer_rmax[r] = c->d_rmax; c->peer_rotflag[r] = c->d_rotflag;
                continue;
            }
            void* p[6] = {};
            for (int i = 0; i < 6 && share; ++i)
                if (i != 2 || c->d_b1) share = open(r, 1 + i, &p[i]);
            c->peer_base[r] = static_cast<float*>(p[0]); c->peer_b0[r] = static_cast<uint8_t*>(p[1]);
            c->peer_b1[r] = static_cast<uint8_t*>(p[2]); c->peer_bnorm[r] = static_cast<uint8_t*>(p[3]);
            c->peer_rmax[r] = static_cast<uint32_t*>(p[4]); c->peer_rotflag[r] = static_cast<unsigned long long*>(p[5]);
        }
    }
    mine.ok = ok;
    mine.share = share ? group : 0;
    rc = gather();                                          // all ranks must agree on the way they exchange
    cudaFree(d_all);
    if (rc) return rc;
    for (uint32_t r = 0; r < W; ++r) { ok = ok && all[r].ok; share = share && all[r].share == group; }
    c->share_group = group;
    c->xchg_on = ok;
    if (!ok) { release_peer_exchange(c); return PINK_B200_OK; }
    c->rot_shared = share && ok;
    if (c->rot_shared) {
        if (!c->bcast_stream) CU_TRY(cudaStreamCreateWithFlags(&c->bcast_stream, cudaStreamNonBlocking));
        for (uint32_t r = 0; r < W; ++r) {
            if (r == rank) continue;
            if (!c->peer_stream[r]) CU_TRY(cudaStreamCreateWithFlags(&c->peer_stream[r], cudaStreamNonBlocking));
            if (!c->peer_sent[r]) CU_TRY(cudaEventCreateWithFlags(&c->peer_sent[r], cudaEventDisableTiming));
        }
        if (!c->share_rotated) CU_TRY(cudaEventCreateWithFlags(&c->share_rotated, cudaEventDisableTiming));
        for (int i = 0; i < 3; ++i)
            if (!c->bcast_done[i]) CU_TRY(cudaEventCreateWithFlags(&c->bcast_done[i], cudaEventDisableTiming));
    }
    return PINK_B200_OK;
}

int train_prepare(pink_b200_ctx* c, uint64_t n)
{
    if (c->failed)
        return fail(PINK_B200_ESTATE, "an earlier device-side wait expired; the context no longer trains (read the map back or destroy it)");
    if (!c->have_som) return fail(PINK_B200_ESTATE, "pink_b200_set_som must be called before training");
    c->af_valid = false;                 // training rewrites the SOM operand: the mapping filter's planes are rebuilt on demand
    if (uses_filter(c) && !c->use_steps) {
        int rcf = ensure_filter_buffers(c, c->filter_imgs ? c->filter_imgs : 1);
        if (rcf) return rcf;
    }
    if (!c->have_factors) return fail(PINK_B200_ESTATE, "pink_b200_set_update_factors must be called before training");
    if (c->cfg.world_size > 1 && !c->comm)
        return fail(PINK_B200_ESTATE, "pink_b200_comm_init must be called before training with world_size > 1");
    int rc = ensure_transform_buffers(c, 2 * kRotBatch, 2 * kRotBatch);
    if (rc) return rc;
    // the persistent kernel exchanges the ranks' records itself, through peer memory only
    c->use_steps = c->plan_ok && c->opt_step_kernel == 0 && c->d_owners && (c->cfg.world_size == 1 || c->xchg_on);
    if (c->bmu_log_cap < n) {
        free_dev(c->d_bmu_log);
        CU_TRY(cudaMalloc(&c->d_bmu_log, n * sizeof(uint32_t)));
        c->bmu_log_cap = n;
    }
    CU_TRY(cudaMemsetAsync(c->d_bmu_log, 0xFF, n * sizeof(uint32_t), c->stream));
    c->bmu_log_n = n;
    return PINK_B200_OK;
}

} // namespace

extern "C" {

const char* pink_b200_last_error(void) { return g_error.c_str(); }

const char* pink_b200_version(void) { return "pink_b200 0.1 (sm_100a)"; }

uint32_t pink_b200_operand_stride(uint32_t K, uint32_t dist_type)
{
    return dist_type == PINK_B200_FLOAT ? round_up(K, 32) : round_up(K, 128);
}

int pink_b200_create(const pink_b200_config* cfg, pink_b200_ctx** out)
{
    if (!cfg || !out) return fail(PINK_B200_EINVAL, "null argument");
    *out = nullptr;
    Geometry g{};
    int rc = make_geometry(*cfg, &g);
    if (rc) return rc;
    if (cfg->world_size == 0 || cfg->rank >= cfg->world_size)
        return fail(PINK_B200_EINVAL, "rank must be smaller than world_size");
    if (cfg->world_size > cfg->n_neurons)
        return fail(PINK_B200_EINVAL, "more neuron shards than neurons");

    CU_TRY(cudaSetDevice(cfg->device));
    cudaDeviceProp prop{};
    CU_TRY(cudaGetDeviceProperties(&prop, cfg->device));
    if (prop.major != 10)
        return fail(PINK_B200_ECUDA, std::string("device '") + prop.name + "' is not an sm_100 GPU; this library has no other code path");

    pink_b200_ctx* c = new (std::nothrow) pink_b200_ctx();
    if (!c) return fail(PINK_B200_EINVAL, "out of host memory");
    c->cfg = *cfg;
    c->g = g;
    const uint32_t W = cfg->world_size, N = cfg->n_neurons;
    const uint32_t base = N / W, extra = N % W;
    c->count = base + (cfg->rank < extra ? 1 : 0);
    // Interleaved shards (rank r holds neurons r, r + W, r + 2W, ...): the neighbourhood of any best matching unit
    // then spreads evenly over the ranks, so every rank has the same share of every image's update.  The sizes are
    // those of the reference's contiguous split (option "sharding" = 1 selects that one).
    c->first = cfg->rank; c->stride = W;
    (void)extra;
    c->train_batch = cfg->max_batch ? cfg->max_batch : 256;
    {
        // Mapping batch: bound the transform operand of one batch to about 1 GiB.
        const size_t per_img = operand_plane_bytes(g, g.T) * (g.mode == kModeU16 ? 2 : 1);
        size_t mb = (size_t(1) << 30) / (per_img ? per_img : 1);
        if (mb < 1) mb = 1;
        if (mb > 64) mb = 64;
        if (cfg->max_batch && mb > cfg->max_batch) mb = cfg->max_batch;
        c->map_batch = (uint32_t)mb;
    }

    auto bail = [&](int code) { pink_b200_destroy(c); return code; };
#define CTX_TRY(expr)                                                                             \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            fail(PINK_B200_ECUDA, std::string(#expr) + ": " + cudaGetErrorString(e_));            \
            return bail(PINK_B200_ECUDA);                                                         \
        }                                                                                         \
    } while (0)

    {
        // The sequential steps run at the highest priority so that their blocks are
        // placed before pending blocks of the look-ahead rotation kernel.
        int lo = 0, hi = 0;
        CTX_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
        CTX_TRY(cudaStreamCreateWithPriority(&c->stream, cudaStreamNonBlocking, hi));
        CTX_TRY(cudaStreamCreateWithPriority(&c->copy_stream, cudaStreamNonBlocking, hi));
        // The rotation kernels (16 images ahead) run on the training stream: on a stream of their own
        // their blocks keep the other kernels' blocks, which need a whole SM each, from starting, and the
        // step gets slower (measured).  Option "rotation_overlap" puts them on a second, low-priority
        // stream anyway; option "step_kernel" selects the older launch sequences.
        c->fuse_update = update_can_fuse(c->g);
        c->rot_stream = c->stream;
        const char* why_not = "";
        c->plan_ok = step_plan(c->g, c->count, N, &c->plan, &why_not);
        if (c->plan_ok) {
            CTX_TRY(cudaMalloc(&c->d_ctrl, sizeof(StepCtrl)));
            CTX_TRY(cudaMalloc(&c->d_owners, (size_t)c->plan.grid * c->plan.owned_per_block * sizeof(uint32_t)));
        }
    }
    for (int i = 0; i < 2; ++i) {
        CTX_TRY(cudaEventCreateWithFlags(&c->copied[i], cudaEventDisableTiming));
        CTX_TRY(cudaEventCreateWithFlags(&c->consumed[i], cudaEventDisableTiming));
        CTX_TRY(cudaEventCreateWithFlags(&c->rotated[i], cudaEventDisableTiming));
        CTX_TRY(cudaEventCreateWithFlags(&c->rot_free[i], cudaEventDisableTiming));
    }
    if (cfg->ed_shape == PINK_B200_CIRCULAR) {
        std::vector<ushort2> spans;
        if (!circle_table(g.nd, g.ed, &spans)) {
            fail(PINK_B200_EINVAL, "circular euclidean distance region does not fit the euclidean distance square");
            return bail(PINK_B200_EINVAL);
        }
        CTX_TRY(cudaMalloc(&c->d_circle, spans.size() * sizeof(ushort2)));
        CTX_TRY(cudaMemcpyAsync(c->d_circle, spans.data(), spans.size() * sizeof(ushort2), cudaMemcpyHostToDevice, c->stream));
        CTX_TRY(cudaStreamSynchronize(c->stream));   // spans goes out of scope
        c->g.circle = c->d_circle;
    }
    CTX_TRY(cudaMalloc(&c->d_som, (size_t)c->count * g.Pp * sizeof(float)));
    CTX_TRY(cudaMemsetAsync(c->d_som, 0, (size_t)c->count * g.Pp * sizeof(float), c->stream));
    CTX_TRY(cudaMalloc(&c->d_a0, operand_plane_bytes(g, c->count)));
    CTX_TRY(cudaMemsetAsync(c->d_a0, 0, operand_plane_bytes(g, c->count), c->stream));
    if (g.mode == kModeU16) {
        CTX_TRY(cudaMalloc(&c->d_a1, operand_plane_bytes(g, c->count)));
        CTX_TRY(cudaMemsetAsync(c->d_a1, 0, operand_plane_bytes(g, c->count), c->stream));
    }
    CTX_TRY(cudaMalloc(&c->d_anorm, norm_bytes(g, c->count)));
    CTX_TRY(cudaMalloc(&c->d_pairs, W * sizeof(BmuPair)));
    CTX_TRY(cudaMemsetAsync(c->d_pairs, 0xFF, W * sizeof(BmuPair), c->stream));
    CTX_TRY(cudaMalloc(&c->d_items, c->count * sizeof(UpdateItem)));
    CTX_TRY(cudaMemsetAsync(c->d_items, 0, c->count * sizeof(UpdateItem), c->stream));
    CTX_TRY(cudaMalloc(&c->d_rmax, 3 * kRotBatch * sizeof(uint32_t)));
    CTX_TRY(cudaMemsetAsync(c->d_rmax, 0, 3 * kRotBatch * sizeof(uint32_t), c->stream));
    CTX_TRY(cudaMalloc(&c->d_stats, 2 * sizeof(unsigned long long)));
    CTX_TRY(cudaMemsetAsync(c->d_stats, 0, 2 * sizeof(unsigned long long), c->stream));
    // [0] work-list length, [1] block arrival counter of the update kernel, [2] of the distance kernel
    CTX_TRY(cudaMalloc(&c->d_nitems, 3 * sizeof(uint32_t)));
    CTX_TRY(cudaMemsetAsync(c->d_nitems, 0, 3 * sizeof(uint32_t), c->stream));
    CTX_TRY(cudaMalloc(&c->d_counts, N * sizeof(uint32_t)));
    CTX_TRY(cudaMemsetAsync(c->d_counts, 0, N * sizeof(uint32_t), c->stream));
    CTX_TRY(cudaMalloc(&c->d_status, sizeof(int)));
    CTX_TRY(cudaMemsetAsync(c->d_status, 0, sizeof(int), c->stream));

    // cos/sin of t * (float(2*pi)/R), t < R/4, evaluated on the host with the
    // reference's expressions (src/SelfOrganizingMapLib/generate_rotated_images.h:70,
    // src/ImageProcessingLib/rotate.h:20-21).
    {
        const uint32_t nq = g.q ? g.q : 1;
        std::vector<float> cs(nq), sn(nq);
        const float step = static_cast<float>(2 * M_PI) / g.R;
        for (uint32_t t = 0; t < nq; ++t) {
            const float angle = t * step;
            cs[t] = std::cos(angle);
            sn[t] = std::sin(angle);
        }
        CTX_TRY(cudaMalloc(&c->d_cs, nq * sizeof(float)));
        CTX_TRY(cudaMalloc(&c->d_sn, nq * sizeof(float)));
        CTX_TRY(cudaMemcpyAsync(c->d_cs, cs.data(), nq * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        CTX_TRY(cudaMemcpyAsync(c->d_sn, sn.data(), nq * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        CTX_TRY(cudaStreamSynchronize(c->stream));   // cs/sn go out of scope
    }
#undef CTX_TRY
    *out = c;
    return PINK_B200_OK;
}

int pink_b200_destroy(pink_b200_ctx* c)
{
    if (!c) return PINK_B200_OK;
    cudaSetDevice(c->cfg.device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->copy_stream) cudaStreamSynchronize(c->copy_stream);
    if (c->rot_stream) cudaStreamSynchronize(c->rot_stream);
    for (uint32_t r = 0; r < kXchgMaxRanks; ++r) if (c->peer_stream[r]) cudaStreamSynchronize(c->peer_stream[r]);
    if (c->bcast_stream) cudaStreamSynchronize(c->bcast_stream);
    release_peer_exchange(c);
    if (c->comm && nccl().ok) nccl().CommDestroy(c->comm);
    free_dev(c->d_som); free_dev(c->d_a0); free_dev(c->d_a1); free_dev(c->d_anorm);
    free_dev(c->d_cs); free_dev(c->d_sn); free_dev(c->d_factors); free_dev(c->d_coords); free_dev(c->d_lut); free_dev(c->d_base);
    free_dev(c->d_b0); free_dev(c->d_b1); free_dev(c->d_bnorm); free_dev(c->d_keys);
    free_dev(c->d_af_hi); free_dev(c->d_af_lo); free_dev(c->d_af_norm); free_dev(c->d_bf_hi); free_dev(c->d_bf_lo);
    free_dev(c->d_bf_norm); free_dev(c->d_est); free_dev(c->d_filter_stats);
    free_dev(c->d_items); free_dev(c->d_nitems); free_dev(c->d_stats); free_dev(c->d_wrange); free_dev(c->d_rmax);
    free_dev(c->d_circle); free_dev(c->d_owners); free_dev(c->d_ctrl); free_dev(c->d_stamps);
    for (cudaEvent_t e : c->prof_launch_events) cudaEventDestroy(e);
    free_dev(c->d_pairs); free_dev(c->d_counts); free_dev(c->d_bmu_log); free_dev(c->d_status);
    free_dev(c->d_images[0]); free_dev(c->d_images[1]); free_dev(c->d_dist); free_dev(c->d_rot);
    for (cudaEvent_t e : c->prof_events) cudaEventDestroy(e);
    for (cudaEvent_t e : c->prof_rot_events) cudaEventDestroy(e);
    for (int i = 0; i < 2; ++i) {
        if (c->copied[i]) cudaEventDestroy(c->copied[i]);
        if (c->consumed[i]) cudaEventDestroy(c->consumed[i]);
        if (c->rotated[i]) cudaEventDestroy(c->rotated[i]);
        if (c->rot_free[i]) cudaEventDestroy(c->rot_free[i]);
    }
    for (uint32_t r = 0; r < kXchgMaxRanks; ++r) {
        if (c->peer_stream[r]) { cudaStreamSynchronize(c->peer_stream[r]); cudaStreamDestroy(c->peer_stream[r]); }
        if (c->peer_sent[r]) cudaEventDestroy(c->peer_sent[r]);
    }
    if (c->bcast_stream) { cudaStreamSynchronize(c->bcast_stream); cudaStreamDestroy(c->bcast_stream); }
    if (c->share_rotated) cudaEventDestroy(c->share_rotated);
    for (int i = 0; i < 3; ++i) if (c->bcast_done[i]) cudaEventDestroy(c->bcast_done[i]);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->rot_stream && c->rot_stream != c->stream) cudaStreamDestroy(c->rot_stream);
    delete c;
    return PINK_B200_OK;
}

int pink_b200_shard(const pink_b200_ctx* c, uint32_t* first, uint32_t* count)
{
    if (!c) return fail(PINK_B200_EINVAL, "null context");
    if (first) *first = c->first;
    if (count) *count = c->count;
    return PINK_B200_OK;
}

uint32_t pink_b200_shard_stride(const pink_b200_ctx* c) { return c ? c->stride : 0; }

int pink_b200_set_option(pink_b200_ctx* c, const char* name, long long value)
{
    if (!c || !name) return fail(PINK_B200_EINVAL, "null argument");
    if (c->have_som || c->comm)
        return fail(PINK_B200_ESTATE, "options must be set before pink_b200_comm_init and pink_b200_set_som");
    const std::string key(name);
    if (key == "step_kernel") {
        if (value < 0 || value > 2) return fail(PINK_B200_EINVAL, "step_kernel must be 0, 1 or 2");
        c->opt_step_kernel = (int)value;
        c->fuse_update = update_can_fuse(c->g) && value != 2;
    } else if (key == "sharding") {
        if (value < 0 || value > 1) return fail(PINK_B200_EINVAL, "sharding must be 0 or 1");
        const uint32_t W = c->cfg.world_size, N = c->cfg.n_neurons, base = N / W, extra = N % W, r = c->cfg.rank;
        if (value == 1) { c->first = r * base + (r < extra ? r : extra); c->stride = 1; }
        else { c->first = r; c->stride = W; }
    } else if (key == "exchange") {
        if (value < 0 || value > 1) return fail(PINK_B200_EINVAL, "exchange must be 0 or 1");
        c->opt_exchange = (int)value;
    } else if (key == "rotation_sharing") {
        if (value < -1 || value == 1) return fail(PINK_B200_EINVAL, "rotation_sharing must be -1, 0 or at least 2");
        c->opt_rotation_sharing = (int)value;
    } else if (key == "rotation_overlap") {
        CU_TRY(cudaSetDevice(c->cfg.device));
        if (value && c->rot_stream == c->stream) {
            int lo = 0, hi = 0;
            CU_TRY(cudaDeviceGetStreamPriorityRange(&lo, &hi));
            CU_TRY(cudaStreamCreateWithPriority(&c->rot_stream, cudaStreamNonBlocking, lo));
        }
    } else if (key == "mma_pairs") {
        c->opt_mma_pairs = value != 0;
    } else if (key == "f32_filter") {
        c->opt_f32_filter = value != 0;
    } else if (key == "cooperative_launch") {
        c->opt_cooperative = value != 0;
    } else if (key == "exchange_timeout_ms") {
        if (value < 1) return fail(PINK_B200_EINVAL, "exchange_timeout_ms must be positive");
        c->opt_exchange_timeout_ms = value;
    } else {
        return fail(PINK_B200_EINVAL, "unknown option '" + key + "'");
    }
    return PINK_B200_OK;
}

int pink_b200_comm_unique_id(void* id128)
{
    if (!id128) return fail(PINK_B200_EINVAL, "null argument");
    if (!nccl().ok) return fail(PINK_B200_ENCCL, "libnccl.so.2 could not be loaded");
    ncclUniqueId id;
    NCCL_TRY(nccl().GetUniqueId(&id));
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    std::memcpy(id128, &id, 128);
    return PINK_B200_OK;
}

int pink_b200_comm_init(pink_b200_ctx* c, const void* id128)
{
    if (!c || !id128) return fail(PINK_B200_EINVAL, "null argument");
    if (c->cfg.world_size == 1) return PINK_B200_OK;
    if (!nccl().ok) return fail(PINK_B200_ENCCL, "libnccl.so.2 could not be loaded");
    if (c->comm) return fail(PINK_B200_ESTATE, "communicator already initialised");
    CU_TRY(cudaSetDevice(c->cfg.device));
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    NCCL_TRY(nccl().CommInitRank(&c->comm, (int)c->cfg.world_size, id, (int)c->cfg.rank));
    return setup_peer_exchange(c);
}

int pink_b200_set_som(pink_b200_ctx* c, const float* host_som)
{
    if (!c || !host_som) return fail(PINK_B200_EINVAL, "null argument");
    const Geometry& g = c->g;
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    // Stream-ordered copy: a blocking cudaMemcpy from pageable memory may return
    // while its DMA is still in flight on the legacy stream, which the
    // context's non-blocking stream does not wait for.
    CU_TRY(cudaMemcpy2DAsync(c->d_som, (size_t)g.Pp * sizeof(float), host_som + (size_t)c->first * g.P,
                             (size_t)c->stride * g.P * sizeof(float), (size_t)g.P * sizeof(float), c->count,
                             cudaMemcpyHostToDevice, c->stream));
    if ((c->fuse_update || c->plan_ok) && !c->d_wrange) CU_TRY(cudaMalloc(&c->d_wrange, (size_t)c->count * sizeof(uint2)));
    LAUNCH_TRY(launch_quantize_som(g, c->d_som, c->count, c->d_a0, c->d_a1, c->d_anorm, c->stream, c->d_wrange));
    c->launches += 1;
    CU_TRY(cudaStreamSynchronize(c->stream));
    c->have_som = true;
    c->af_valid = false;
    return PINK_B200_OK;
}

int pink_b200_get_som(pink_b200_ctx* c, float* host_som)
{
    if (!c || !host_som) return fail(PINK_B200_EINVAL, "null argument");
    const Geometry& g = c->g;
    CU_TRY(cudaSetDevice(c->cfg.device));
    int rc = check_status(c);
    if (rc) return rc;
    CU_TRY(cudaMemcpy2DAsync(host_som + (size_t)c->first * g.P, (size_t)c->stride * g.P * sizeof(float), c->d_som,
                             (size_t)g.Pp * sizeof(float), (size_t)g.P * sizeof(float), c->count,
                             cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    return PINK_B200_OK;
}

int pink_b200_set_update_factors(pink_b200_ctx* c, const float* host_factors)
{
    if (!c || !host_factors) return fail(PINK_B200_EINVAL, "null argument");
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    const size_t N = c->cfg.n_neurons;
    free_dev(c->d_lut);
    if (!c->d_factors) CU_TRY(cudaMalloc(&c->d_factors, N * c->count * sizeof(float)));
    {
        // this shard's columns of the table, gathered on the host: F[b][first + j * stride]
        std::vector<float> cols(N * c->count);
        for (size_t b = 0; b < N; ++b) {
            const float* row = host_factors + b * N + c->first;
            float* out = cols.data() + b * c->count;
            for (size_t j = 0; j < c->count; ++j) out[j] = row[j * c->stride];
        }
        CU_TRY(cudaMemcpyAsync(c->d_factors, cols.data(), cols.size() * sizeof(float), cudaMemcpyHostToDevice, c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));
    }
    if (c->plan_ok) {
        // which block of the persistent kernel rewrites which neuron: spread every neighbourhood over the blocks
        std::vector<uint32_t> owners((size_t)c->plan.grid * c->plan.owned_per_block);
        step_assign_owners([&](uint32_t i, uint32_t m) { return host_factors[(size_t)i * N + m]; }, c->first, c->stride,
                           c->count, c->plan, owners.data());
        CU_TRY(cudaMemcpyAsync(c->d_owners, owners.data(), owners.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));
    }
    c->factor_source = FactorSource{};
    c->factor_source.table = c->d_factors;
    c->have_factors = true;
    return PINK_B200_OK;
}

int pink_b200_set_update_lut(pink_b200_ctx* c, uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                             const float* host_lut, uint32_t n_classes)
{
    if (!c || !host_lut) return fail(PINK_B200_EINVAL, "null argument");
    const uint32_t want = pink_b200_distance_classes(som_layout, dim0, dim1, dim2, nullptr, 0);
    if (want == 0 || want != n_classes) return fail(PINK_B200_EINVAL, "the table does not have one entry per distance class of this SOM layout");
    const uint32_t N = c->cfg.n_neurons;
    const uint64_t size = som_layout == PINK_B200_LAYOUT_HEXAGONAL ? pink_b200_som_size(som_layout, dim0, dim1)
                                                                   : (uint64_t)dim0 * dim1 * dim2;
    if (size != N) return fail(PINK_B200_EINVAL, "the SOM layout does not have the context's number of neurons");
    std::vector<int16_t> coords((size_t)4 * N);
    if (pink_b200_som_coordinates(som_layout, dim0, dim1, dim2, coords.data()) != PINK_B200_OK)
        return fail(PINK_B200_EINVAL, "unsupported SOM layout");
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    free_dev(c->d_factors); free_dev(c->d_lut);
    if (!c->d_coords) CU_TRY(cudaMalloc(&c->d_coords, (size_t)N * sizeof(short4)));
    CU_TRY(cudaMalloc(&c->d_lut, (size_t)n_classes * sizeof(float)));
    CU_TRY(cudaMemcpyAsync(c->d_coords, coords.data(), (size_t)N * sizeof(short4), cudaMemcpyHostToDevice, c->stream));
    CU_TRY(cudaMemcpyAsync(c->d_lut, host_lut, (size_t)n_classes * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    const bool hex = som_layout == PINK_B200_LAYOUT_HEXAGONAL;
    if (c->plan_ok) {
        auto cls = [&](uint32_t i, uint32_t m) -> uint32_t {
            const int dx = coords[4 * i] - coords[4 * m], dy = coords[4 * i + 1] - coords[4 * m + 1], dz = coords[4 * i + 2] - coords[4 * m + 2];
            if (hex) return ((dx >= 0) == (dy >= 0)) ? (uint32_t)std::abs(dx + dy) : (uint32_t)std::max(std::abs(dx), std::abs(dy));
            return ((uint32_t)std::abs(dz) * dim0 + (uint32_t)std::abs(dy)) * dim1 + (uint32_t)std::abs(dx);
        };
        std::vector<uint32_t> owners((size_t)c->plan.grid * c->plan.owned_per_block);
        step_assign_owners([&](uint32_t i, uint32_t m) { return host_lut[cls(i, m)]; }, c->first, c->stride, c->count, c->plan,
                           owners.data());
        CU_TRY(cudaMemcpyAsync(c->d_owners, owners.data(), owners.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
        CU_TRY(cudaStreamSynchronize(c->stream));
    }
    c->factor_source = FactorSource{};
    c->factor_source.coords = c->d_coords;
    c->factor_source.lut = c->d_lut;
    c->factor_source.hexagonal = hex;
    c->factor_source.dim0 = dim0; c->factor_source.dim1 = dim1;
    c->have_factors = true;
    return PINK_B200_OK;
}

int pink_b200_set_update_function(pink_b200_ctx* c, uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                  uint32_t func, float p0, float p1, float max_update_distance)
{
    if (!c) return fail(PINK_B200_EINVAL, "null argument");
    const uint32_t n = pink_b200_distance_classes(som_layout, dim0, dim1, dim2, nullptr, 0);
    if (n == 0) return fail(PINK_B200_EINVAL, "unsupported SOM layout");
    std::vector<float> lut(n);
    if (pink_b200_update_lut(som_layout, dim0, dim1, dim2, func, p0, p1, max_update_distance, lut.data(), n) != PINK_B200_OK)
        return fail(PINK_B200_EINVAL, "unsupported neighbourhood function");
    return pink_b200_set_update_lut(c, som_layout, dim0, dim1, dim2, lut.data(), n);
}

int pink_b200_train_device(pink_b200_ctx* c, const float* dev_images, uint64_t n)
{
    if (!c || (!dev_images && n)) return fail(PINK_B200_EINVAL, "null argument");
    CU_TRY(cudaSetDevice(c->cfg.device));
    int rc = train_prepare(c, n);
    if (rc) return rc;
    rc = train_chunk(c, dev_images, n, c->d_bmu_log, nullptr);
    if (rc) return rc;
    CU_TRY(cudaGetLastError());
    return PINK_B200_OK;
}

int pink_b200_train(pink_b200_ctx* c, const float* host_images, uint64_t n)
{
    if (!c || (!host_images && n)) return fail(PINK_B200_EINVAL, "null argument");
    CU_TRY(cudaSetDevice(c->cfg.device));
    int rc = train_prepare(c, n);
    if (rc) return rc;
    const size_t B = c->train_batch, isz = c->image_size();
    rc = ensure_image_staging(c, B > c->map_batch ? B : c->map_batch);
    if (rc) return rc;
    // Double-buffered staging: the copy of batch k+1 overlaps the steps of batch k.
    uint64_t done = 0;
    for (uint64_t k = 0; done < n; ++k) {
        const int buf = (int)(k & 1);
        const uint64_t m = n - done < B ? n - done : B;
        CU_TRY(cudaStreamWaitEvent(c->copy_stream, c->consumed[buf], 0));
        CU_TRY(cudaMemcpyAsync(c->d_images[buf], host_images + done * isz, m * isz * sizeof(float),
                               cudaMemcpyHostToDevice, c->copy_stream));
        CU_TRY(cudaEventRecord(c->copied[buf], c->copy_stream));
        rc = train_chunk(c, c->d_images[buf], m, c->d_bmu_log + done, c->copied[buf]);
        if (rc) return rc;
        CU_TRY(cudaEventRecord(c->consumed[buf], c->stream));
        done += m;
    }
    CU_TRY(cudaGetLastError());
    return PINK_B200_OK;
}

int pink_b200_get_update_counts(pink_b200_ctx* c, uint32_t* host_counts)
{
    if (!c || !host_counts) return fail(PINK_B200_EINVAL, "null argument");
    CU_TRY(cudaSetDevice(c->cfg.device));
    int rc = check_status(c);
    if (rc) return rc;
    CU_TRY(cudaMemcpyAsync(host_counts, c->d_counts, (size_t)c->cfg.n_neurons * sizeof(uint32_t),
                           cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    return PINK_B200_OK;
}

int pink_b200_get_bmu_log(pink_b200_ctx* c, uint32_t* host_bmus, uint64_t n)
{
    if (!c || !host_bmus) return fail(PINK_B200_EINVAL, "null argument");
    if (n > c->bmu_log_n) return fail(PINK_B200_EINVAL, "more entries requested than the last train call produced");
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaMemcpyAsync(host_bmus, c->d_bmu_log, n * sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    return PINK_B200_OK;
}

static int map_chunk(pink_b200_ctx* c, const float* d_images, uint32_t m, float* d_dist, uint32_t* d_rot)
{
    const Geometry& g = c->g;
    const bool filter = uses_filter(c);
    if (filter) {
        int rc = ensure_filter_buffers(c, c->map_batch);
        if (rc) return rc;
        // the rotation kernel also writes the estimate's TF32 planes and norms of the transforms
        LAUNCH_TRY(launch_rotate(g, d_images, m, c->d_cs, c->d_sn, base_fits_smem(g) ? nullptr : c->d_base, c->d_b0, c->d_bf_hi,
                                 c->d_bf_norm, c->stream, nullptr, c->d_bf_lo));
    } else {
        LAUNCH_TRY(launch_rotate(g, d_images, m, c->d_cs, c->d_sn, base_fits_smem(g) ? nullptr : c->d_base, c->d_b0, c->d_b1, c->d_bnorm, c->stream));
    }
    DistanceArgs da{};
    da.a0 = c->d_a0; da.a1 = c->d_a1; da.anorm = c->d_anorm; da.n = c->count;
    da.b0 = c->d_b0; da.b1 = c->d_b1; da.bnorm = c->d_bnorm; da.n_img = m;
    da.keys = c->d_keys; da.s_out = nullptr; da.status = c->d_status; da.single_cta = !c->opt_mma_pairs;
    const char* why = "";
    if (filter) {
        // estimate of every pair on the tensor cores, then exact sums for the transforms it cannot rule out
        const float* A = static_cast<const float*>(c->d_a0);
        const float* B = static_cast<const float*>(c->d_b0);
        if (!c->af_valid) {
            LAUNCH_TRY(launch_split_tf32(A, c->count, g.Kp, c->d_af_hi, c->d_af_lo, c->d_af_norm, c->stream));
            c->af_valid = true;
            c->launches += 1;
        }
        da.a0 = c->d_af_hi; da.a1 = c->d_af_lo; da.anorm = c->d_af_norm;
        da.b0 = c->d_bf_hi; da.b1 = c->d_bf_lo; da.bnorm = c->d_bf_norm;
        da.s_out = c->d_est;
        cudaError_t e = launch_distance_tf32(g, da, c->stream, &why);
        if (e != cudaSuccess) return fail(PINK_B200_ECUDA, std::string(why) + ": " + cudaGetErrorString(e));
        const float eps = filter_eps(g.K);
        LAUNCH_TRY(launch_refine_f32(g, A, c->d_af_norm, c->count, B, c->d_bf_norm, m, c->d_est, eps, c->d_keys,
                                     c->d_filter_stats, c->stream));
        c->filter_pairs += (unsigned long long)m * c->count * g.T;
        LAUNCH_TRY(launch_map_finalize(g, c->d_keys, m, c->count, d_dist, d_rot, c->stream));
        c->launches += 4;                 // rotation set, estimate, exact pass, epilogue
        return PINK_B200_OK;
    }
    cudaError_t e = launch_distance(g, da, c->stream, &why);
    if (e != cudaSuccess) return fail(PINK_B200_ECUDA, std::string(why) + ": " + cudaGetErrorString(e));
    LAUNCH_TRY(launch_map_finalize(g, c->d_keys, m, c->count, d_dist, d_rot, c->stream));
    c->launches += 3;                 // rotation set, distance, epilogue
    return PINK_B200_OK;
}

int pink_b200_map_filter_stats(pink_b200_ctx* c, double out[4])
{
    if (!c || !out) return fail(PINK_B200_EINVAL, "null argument");
    out[0] = (double)c->filter_pairs; out[1] = 0.0; out[2] = 0.0;
    out[3] = (double)filter_eps(c->g.K);
    if (!c->d_filter_stats) return PINK_B200_OK;
    CU_TRY(cudaSetDevice(c->cfg.device));
    unsigned long long h[2] = { 0, 0 };
    CU_TRY(cudaMemcpyAsync(h, c->d_filter_stats, sizeof(h), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    const uint32_t bits = (uint32_t)h[1];
    float worst;
    std::memcpy(&worst, &bits, sizeof(worst));
    out[1] = (double)h[0];
    out[2] = (double)worst;
    return PINK_B200_OK;
}

int pink_b200_map_device(pink_b200_ctx* c, const float* dev_images, uint64_t n, float* dev_dist, uint32_t* dev_rot)
{
    if (!c || ((!dev_images || !dev_dist || !dev_rot) && n)) return fail(PINK_B200_EINVAL, "null argument");
    if (!c->have_som) return fail(PINK_B200_ESTATE, "pink_b200_set_som must be called before mapping");
    CU_TRY(cudaSetDevice(c->cfg.device));
    int rc = ensure_transform_buffers(c, c->map_batch, base_fits_smem(c->g) ? 0 : c->map_batch);
    if (rc) return rc;
    for (uint64_t done = 0; done < n;) {
        const uint32_t m = (uint32_t)(n - done < c->map_batch ? n - done : c->map_batch);
        rc = map_chunk(c, dev_images + done * c->image_size(), m, dev_dist + done * c->count, dev_rot + done * c->count);
        if (rc) return rc;
        done += m;
    }
    CU_TRY(cudaGetLastError());
    return PINK_B200_OK;
}

int pink_b200_map(pink_b200_ctx* c, const float* host_images, uint64_t n, float* host_dist, uint32_t* host_rot)
{
    if (!c || ((!host_images || !host_dist || !host_rot) && n)) return fail(PINK_B200_EINVAL, "null argument");
    if (!c->have_som) return fail(PINK_B200_ESTATE, "pink_b200_set_som must be called before mapping");
    CU_TRY(cudaSetDevice(c->cfg.device));
    const size_t B = c->map_batch, isz = c->image_size();
    int rc = ensure_transform_buffers(c, B, base_fits_smem(c->g) ? 0 : B);
    if (rc) return rc;
    rc = ensure_image_staging(c, B > c->train_batch ? B : c->train_batch);
    if (rc) return rc;
    if (c->out_imgs < 2 * B) {
        free_dev(c->d_dist); free_dev(c->d_rot);
        CU_TRY(cudaMalloc(&c->d_dist, 2 * B * c->count * sizeof(float)));
        CU_TRY(cudaMalloc(&c->d_rot, 2 * B * c->count * sizeof(uint32_t)));
        c->out_imgs = 2 * B;
    }
    // Batches alternate between two staging/result buffers: the upload of batch
    // k+1 and the download of batch k-1 overlap the kernels of batch k.
    uint64_t done = 0;
    for (uint64_t k = 0; done < n; ++k) {
        const int buf = (int)(k & 1);
        const uint32_t m = (uint32_t)(n - done < B ? n - done : B);
        float* dd = c->d_dist + (size_t)buf * B * c->count;
        uint32_t* dr = c->d_rot + (size_t)buf * B * c->count;
        CU_TRY(cudaStreamWaitEvent(c->copy_stream, c->consumed[buf], 0));
        CU_TRY(cudaMemcpyAsync(c->d_images[buf], host_images + done * isz, m * isz * sizeof(float),
                               cudaMemcpyHostToDevice, c->copy_stream));
        CU_TRY(cudaEventRecord(c->copied[buf], c->copy_stream));
        CU_TRY(cudaStreamWaitEvent(c->stream, c->copied[buf], 0));
        rc = map_chunk(c, c->d_images[buf], m, dd, dr);
        if (rc) return rc;
        CU_TRY(cudaMemcpyAsync(host_dist + done * c->count, dd, (size_t)m * c->count * sizeof(float),
                               cudaMemcpyDeviceToHost, c->stream));
        CU_TRY(cudaMemcpyAsync(host_rot + done * c->count, dr, (size_t)m * c->count * sizeof(uint32_t),
                               cudaMemcpyDeviceToHost, c->stream));
        CU_TRY(cudaEventRecord(c->consumed[buf], c->stream));
        done += m;
    }
    return check_status(c);
}

int pink_b200_synchronize(pink_b200_ctx* c)
{
    if (!c) return fail(PINK_B200_EINVAL, "null context");
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->copy_stream));
    CU_TRY(cudaStreamSynchronize(c->rot_stream));
    return check_status(c);
}

void* pink_b200_stream(pink_b200_ctx* c) { return c ? c->stream : nullptr; }

uint64_t pink_b200_launch_count(pink_b200_ctx* c) { return c ? c->launches : 0; }

int pink_b200_exchange_kind(pink_b200_ctx* c)
{
    if (!c || c->cfg.world_size == 1 || !c->comm) return PINK_B200_EXCHANGE_NONE;
    if (c->rot_shared) return PINK_B200_EXCHANGE_PEER_SHARED_ROTATION;
    return c->xchg_on ? PINK_B200_EXCHANGE_PEER : PINK_B200_EXCHANGE_NCCL;
}

int pink_b200_get_update_stats(pink_b200_ctx* c, uint64_t* out)
{
    if (!c || !out) return fail(PINK_B200_EINVAL, "null argument");
    CU_TRY(cudaSetDevice(c->cfg.device));
    unsigned long long v[2] = {0, 0};
    CU_TRY(cudaMemcpyAsync(v, c->d_stats, sizeof(v), cudaMemcpyDeviceToHost, c->stream));
    CU_TRY(cudaStreamSynchronize(c->stream));
    out[0] = v[0]; out[1] = v[1];
    return PINK_B200_OK;
}

int pink_b200_profile_begin(pink_b200_ctx* c, uint32_t max_steps)
{
    if (!c) return fail(PINK_B200_EINVAL, "null context");
    CU_TRY(cudaSetDevice(c->cfg.device));
    while (c->prof_events.size() < (size_t)4 * max_steps) {
        cudaEvent_t e;
        CU_TRY(cudaEventCreate(&e));
        c->prof_events.push_back(e);
    }
    while (c->prof_rot_events.size() < (size_t)2 * (max_steps / kRotBatch + 2)) {
        cudaEvent_t e;
        CU_TRY(cudaEventCreate(&e));
        c->prof_rot_events.push_back(e);
    }
    while (c->prof_launch_events.size() < (size_t)2 * (max_steps / kRotBatch + 2)) {
        cudaEvent_t e;
        CU_TRY(cudaEventCreate(&e));
        c->prof_launch_events.push_back(e);
    }
    if (c->plan_ok && c->stamps_cap < max_steps) {
        free_dev(c->d_stamps);
        CU_TRY(cudaMalloc(&c->d_stamps, (size_t)max_steps * c->plan.grid * kStepStampWords * sizeof(unsigned long long)));
        c->stamps_cap = max_steps;
    }
    if (c->d_stamps) CU_TRY(cudaMemsetAsync(c->d_stamps, 0, c->stamps_cap * c->plan.grid * kStepStampWords * sizeof(unsigned long long), c->stream));
    c->prof_cap = max_steps;
    c->prof_used = c->prof_rot_used = 0;
    c->prof_launches = c->prof_launch_images = 0;
    return PINK_B200_OK;
}

int pink_b200_profile_end(pink_b200_ctx* c, double ms_sum[4], uint64_t* steps)
{
    if (!c || !ms_sum || !steps) return fail(PINK_B200_EINVAL, "null argument");
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    CU_TRY(cudaStreamSynchronize(c->rot_stream));
    for (int k = 0; k < 4; ++k) ms_sum[k] = 0.0;
    for (size_t s = 0; s < c->prof_rot_used; ++s) {
        float ms = 0.f;
        CU_TRY(cudaEventElapsedTime(&ms, c->prof_rot_events[2 * s], c->prof_rot_events[2 * s + 1]));
        ms_sum[0] += ms;
    }
    if (c->use_steps) {
        // persistent kernel: the phases of a step are read from block 0's device-timer stamps
        const size_t per_step = (size_t)kStepStampWords * c->plan.grid;
        std::vector<unsigned long long> t(per_step * c->prof_used);
        if (c->prof_used) CU_TRY(cudaMemcpy(t.data(), c->d_stamps, t.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
        for (size_t s = 0; s < c->prof_used; ++s) {
            const unsigned long long* q = &t[per_step * s];
            ms_sum[1] += (double)(q[2] - q[0]) * 1e-6;      // distance phase up to the first grid barrier
            ms_sum[2] += (double)(q[3] - q[2]) * 1e-6;      // best matching unit (+ exchange) and work list
            ms_sum[3] += (double)(q[5] - q[3]) * 1e-6;      // update phase up to the second grid barrier
        }
    } else {
        for (size_t s = 0; s < c->prof_used; ++s)
            for (int k = 0; k < 3; ++k) {
                float ms = 0.f;
                CU_TRY(cudaEventElapsedTime(&ms, c->prof_events[4 * s + k], c->prof_events[4 * s + k + 1]));
                ms_sum[k + 1] += ms;
            }
    }
    *steps = c->prof_used;
    c->prof_cap = 0;                   // prof_used and the stamps stay readable for pink_b200_profile_detail
    return PINK_B200_OK;
}

int pink_b200_profile_detail(pink_b200_ctx* c, double out[8])
{
    if (!c || !out) return fail(PINK_B200_EINVAL, "null argument");
    for (int k = 0; k < 8; ++k) out[k] = 0.0;
    if (!c->use_steps || c->prof_used == 0 || c->prof_launches == 0) return PINK_B200_OK;
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    double ms_total = 0.0;
    for (size_t l = 0; l < c->prof_launches; ++l) {
        float ms = 0.f;
        CU_TRY(cudaEventElapsedTime(&ms, c->prof_launch_events[2 * l], c->prof_launch_events[2 * l + 1]));
        ms_total += ms;
    }
    out[0] = 1e3 * ms_total / (double)c->prof_launches;
    out[1] = (double)c->prof_launch_images / (double)c->prof_launches;
    const size_t per_step = (size_t)kStepStampWords * c->plan.grid;
    std::vector<unsigned long long> t(per_step * c->prof_used);
    CU_TRY(cudaMemcpy(t.data(), c->d_stamps, t.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    for (size_t s = 0; s < c->prof_used; ++s)
        for (int k = 0; k < 5; ++k)
            out[2 + k] += (double)(t[per_step * s + k + 1] - t[per_step * s + k]) * 1e-3 / (double)c->prof_used;
    return PINK_B200_OK;
}

int pink_b200_profile_stamps(pink_b200_ctx* c, uint64_t* out, uint64_t capacity, uint32_t* blocks, uint64_t* steps)
{
    if (!c || !blocks || !steps) return fail(PINK_B200_EINVAL, "null argument");
    *blocks = c->use_steps ? c->plan.grid : 0;
    *steps = c->use_steps ? c->prof_used : 0;
    const uint64_t words = (uint64_t)kStepStampWords * *blocks * *steps;
    if (!out || words == 0) return PINK_B200_OK;
    if (capacity < words) return fail(PINK_B200_EINVAL, "buffer too small for the stamps");
    CU_TRY(cudaSetDevice(c->cfg.device));
    CU_TRY(cudaStreamSynchronize(c->stream));
    CU_TRY(cudaMemcpy(out, c->d_stamps, words * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return PINK_B200_OK;
}

// ---- single stages ---------------------------------------------------------------

// device status word of the single-stage entries, one per device (a kernel may only be handed memory of its own GPU)
constexpr int kOpMaxDevices = 64;
static std::atomic<int*> g_op_status[kOpMaxDevices];

static int op_status_word(int** out)
{
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kOpMaxDevices) return fail(PINK_B200_EINVAL, "device ordinal out of range");
    int* p = g_op_status[dev].load(std::memory_order_acquire);
    if (!p) {
        int* fresh = nullptr;
        CU_TRY(cudaMalloc(&fresh, sizeof(int)));
        CU_TRY(cudaMemset(fresh, 0, sizeof(int)));
        if (g_op_status[dev].compare_exchange_strong(p, fresh, std::memory_order_acq_rel)) p = fresh;
        else cudaFree(fresh);                      // another thread was first
    }
    *out = p;
    return PINK_B200_OK;
}

static int stage_tables(const Geometry& g, float** d_cs, float** d_sn, cudaStream_t st)
{
    const uint32_t nq = g.q ? g.q : 1;
    std::vector<float> cs(nq), sn(nq);
    const float step = static_cast<float>(2 * M_PI) / g.R;
    for (uint32_t t = 0; t < nq; ++t) { const float a = t * step; cs[t] = std::cos(a); sn[t] = std::sin(a); }
    *d_cs = *d_sn = nullptr;
    cudaError_t e = cudaMalloc(d_cs, nq * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(d_sn, nq * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpyAsync(*d_cs, cs.data(), nq * sizeof(float), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(*d_sn, sn.data(), nq * sizeof(float), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        cudaFree(*d_cs); cudaFree(*d_sn);          // nothing leaks on the error paths
        *d_cs = *d_sn = nullptr;
        return fail(PINK_B200_ECUDA, std::string("staging the rotation tables: ") + cudaGetErrorString(e));
    }
    return PINK_B200_OK;
}

int pink_b200_op_rotate(const pink_b200_config* cfg, const float* dev_images, uint32_t n_img,
                        float* dev_base, void* dev_b0, void* dev_b1, void* dev_bnorm, void* stream)
{
    if (!cfg || !dev_images || !dev_b0) return fail(PINK_B200_EINVAL, "null argument");
    Geometry g{};
    int rc = geometry_from_config(cfg, &g);
    if (rc) return rc;
    if (!dev_base && (size_t)g.P * sizeof(float) > 200 * 1024)
        return fail(PINK_B200_EINVAL, "dev_base is required when a base rotation does not fit shared memory");
    float *d_cs = nullptr, *d_sn = nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = stage_tables(g, &d_cs, &d_sn, st);
    if (rc) return rc;
    cudaError_t e = launch_rotate(g, dev_images, n_img, d_cs, d_sn, dev_base, dev_b0, dev_b1, dev_bnorm, st);
    cudaStreamSynchronize(st);
    cudaFree(d_cs); cudaFree(d_sn);
    if (e != cudaSuccess) return fail(PINK_B200_ECUDA, std::string("rotate_kernel launch: ") + cudaGetErrorString(e));
    return PINK_B200_OK;
}

int pink_b200_op_quantize_som(const pink_b200_config* cfg, const float* dev_som, uint32_t n_neurons,
                              void* dev_a0, void* dev_a1, void* dev_anorm, void* stream)
{
    if (!cfg || !dev_som || !dev_a0) return fail(PINK_B200_EINVAL, "null argument");
    Geometry g{};
    int rc = geometry_from_config(cfg, &g);
    if (rc) return rc;
    if (g.P != g.Pp) return fail(PINK_B200_EINVAL, "this entry needs a neuron size that is a multiple of 4 floats");
    LAUNCH_TRY(launch_quantize_som(g, dev_som, n_neurons, dev_a0, dev_a1, dev_anorm, static_cast<cudaStream_t>(stream)));
    return PINK_B200_OK;
}

int pink_b200_op_distance(uint32_t dist_type, uint32_t n_neurons, uint32_t n_transforms, uint32_t K,
                          const void* dev_a0, const void* dev_a1, const void* dev_anorm,
                          const void* dev_b0, const void* dev_b1, const void* dev_bnorm, uint32_t n_img,
                          unsigned long long* dev_keys, void* dev_matrix, void* stream)
{
    if (!dev_a0 || !dev_b0 || !dev_keys) return fail(PINK_B200_EINVAL, "null argument");
    if (dist_type > PINK_B200_UINT8) return fail(PINK_B200_EINVAL, "Unknown euclidean_distance_type");
    if (dist_type != PINK_B200_FLOAT && (!dev_anorm || !dev_bnorm)) return fail(PINK_B200_EINVAL, "null norm argument");
    if (dist_type == PINK_B200_UINT16 && (!dev_a1 || !dev_b1)) return fail(PINK_B200_EINVAL, "null low-byte plane");
    if (dist_type == PINK_B200_UINT8 && K > 33025) return fail(PINK_B200_EINVAL, "uint8 distance supports at most 33025 elements");
    if (dist_type == PINK_B200_UINT16 && K > 16512) return fail(PINK_B200_EINVAL, "uint16 distance supports at most 16512 elements");
    Geometry g{};
    g.mode = (int)dist_type;
    g.T = n_transforms; g.K = K; g.Kp = pink_b200_operand_stride(K, dist_type);
    int* d_status = nullptr;
    {
        const int rc = op_status_word(&d_status);
        if (rc) return rc;
    }
    DistanceArgs da{};
    da.a0 = dev_a0; da.a1 = dev_a1; da.anorm = dev_anorm; da.n = n_neurons;
    da.b0 = dev_b0; da.b1 = dev_b1; da.bnorm = dev_bnorm; da.n_img = n_img;
    da.keys = dev_keys; da.s_out = dev_matrix; da.status = d_status;
    const char* why = "";
    cudaError_t e = launch_distance(g, da, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess) return fail(PINK_B200_ECUDA, std::string(why) + ": " + cudaGetErrorString(e));
    return PINK_B200_OK;
}

int pink_b200_op_status(void)
{
    int dev = 0;
    CU_TRY(cudaGetDevice(&dev));
    int* word = (dev >= 0 && dev < kOpMaxDevices) ? g_op_status[dev].load(std::memory_order_acquire) : nullptr;
    if (!word) return PINK_B200_OK;
    int st = 0;
    CU_TRY(cudaDeviceSynchronize());
    CU_TRY(cudaMemcpy(&st, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (st != kDevOk) {
        cudaMemset(word, 0, sizeof(int));
        return fail(PINK_B200_ETIMEOUT, "a bounded device-side wait expired (code " + std::to_string(st) + ")");
    }
    return PINK_B200_OK;
}

} // extern "C"
