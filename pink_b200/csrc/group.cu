// One process driving several GPUs: what the reference's Trainer / Mapper do on their own when more than one
// GPU is visible (src/CudaLib/CudaLib.cu:56-76 lists the devices,
// src/CudaLib/generate_euclidean_distance_matrix_first_step_multi_gpu.h:47-196 splits the neurons over them with
// one host thread per extra GPU).  A group owns
//   - for training: one neuron-shard context per device (rank r on devices[r]); the shards' records are exchanged
//     through peer memory exactly as between processes, the contexts are driven by one host thread each;
//   - for mapping: one whole-SOM context per device; the images of a call are dealt to the devices in contiguous
//     ranges and the results land in file order (mapping needs no communication at all).
// Host code only; every device-side step goes through the single-context entry points.
#include "../../include/pink_b200.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <functional>
#include <new>
#include <string>
#include <thread>
#include <vector>

namespace pinkb {
int report_error(int code, const char* msg);
}

struct pink_b200_group
{
    pink_b200_config cfg{};
    std::vector<int32_t> devices;
    std::vector<pink_b200_ctx*> train;      // neuron shards (world = number of devices), created on first use
    std::vector<pink_b200_ctx*> map;        // whole-SOM contexts, created on first use (one device: the training context)
    std::vector<std::pair<std::string, long long>> options;
    std::vector<float> som;                 // host copy of the whole map: source for contexts created later
    std::vector<float> factors;             // N x N table, or (lut_layout[0] != ~0u) one value per distance class
    uint32_t lut_layout[4] = {~0u, 0, 0, 0};
    bool have_som = false, have_factors = false;
    bool train_has_som = false, train_has_factors = false, map_has_som = false;
    bool som_stale = false;                 // the training contexts hold a newer map than `som`
};

namespace {

using pinkb::report_error;

// Runs fn(d) for every device index in its own host thread (the calling thread takes index 0) and returns the first
// failure.  Error messages are per thread, so the failing thread's message is carried over to the caller.
int for_each_device(size_t n, const std::function<int(size_t)>& fn)
{
    std::vector<int> rc(n, PINK_B200_OK);
    std::vector<std::string> msg(n);
    auto run = [&](size_t d) {
        rc[d] = fn(d);
        if (rc[d] != PINK_B200_OK) msg[d] = pink_b200_last_error();
    };
    std::vector<std::thread> threads;
    for (size_t d = 1; d < n; ++d) threads.emplace_back(run, d);
    run(0);
    for (std::thread& t : threads) t.join();
    for (size_t d = 0; d < n; ++d)
        if (rc[d] != PINK_B200_OK) return report_error(rc[d], msg[d].c_str());
    return PINK_B200_OK;
}

int apply_options(const pink_b200_group* g, pink_b200_ctx* c)
{
    for (const auto& o : g->options) {
        const int rc = pink_b200_set_option(c, o.first.c_str(), o.second);
        if (rc != PINK_B200_OK) return rc;
    }
    return PINK_B200_OK;
}

// The training contexts: created, connected and loaded with the current map and factors.
int ensure_train(pink_b200_group* g)
{
    const size_t W = g->devices.size();
    if (g->train.empty()) {
        g->train.assign(W, nullptr);
        unsigned char id[128] = {};
        if (W > 1) {
            const int rc = pink_b200_comm_unique_id(id);
            if (rc != PINK_B200_OK) return rc;
        }
        int rc = for_each_device(W, [&](size_t d) {
            pink_b200_config cfg = g->cfg;
            cfg.device = g->devices[d]; cfg.rank = (uint32_t)d; cfg.world_size = (uint32_t)W;
            int r = pink_b200_create(&cfg, &g->train[d]);
            if (r == PINK_B200_OK) r = apply_options(g, g->train[d]);
            if (r == PINK_B200_OK && W > 1) r = pink_b200_comm_init(g->train[d], id);      // collective: all threads take part
            return r;
        });
        if (rc != PINK_B200_OK) return rc;
    }
    if (!g->train_has_som && g->have_som) {
        int rc = for_each_device(W, [&](size_t d) { return pink_b200_set_som(g->train[d], g->som.data()); });
        if (rc != PINK_B200_OK) return rc;
        g->train_has_som = true;
    }
    if (!g->train_has_factors && g->have_factors) {
        int rc = for_each_device(W, [&](size_t d) {
            if (g->lut_layout[0] == ~0u) return pink_b200_set_update_factors(g->train[d], g->factors.data());
            return pink_b200_set_update_lut(g->train[d], g->lut_layout[0], g->lut_layout[1], g->lut_layout[2], g->lut_layout[3],
                                            g->factors.data(), (uint32_t)g->factors.size());
        });
        if (rc != PINK_B200_OK) return rc;
        g->train_has_factors = true;
    }
    return PINK_B200_OK;
}

// Brings the host copy of the map up to date with the training contexts.
int refresh_som(pink_b200_group* g)
{
    if (!g->som_stale) return PINK_B200_OK;
    int rc = for_each_device(g->train.size(), [&](size_t d) { return pink_b200_get_som(g->train[d], g->som.data()); });
    if (rc != PINK_B200_OK) return rc;
    g->som_stale = false;
    g->map_has_som = false;
    return PINK_B200_OK;
}

int ensure_map(pink_b200_group* g)
{
    const size_t W = g->devices.size();
    int rc = refresh_som(g);
    if (rc != PINK_B200_OK) return rc;
    if (g->map.empty()) {
        g->map.assign(W, nullptr);
        rc = for_each_device(W, [&](size_t d) {
            pink_b200_config cfg = g->cfg;
            cfg.device = g->devices[d]; cfg.rank = 0; cfg.world_size = 1;
            return pink_b200_create(&cfg, &g->map[d]);
        });
        if (rc != PINK_B200_OK) return rc;
    }
    if (!g->map_has_som) {
        rc = for_each_device(W, [&](size_t d) { return pink_b200_set_som(g->map[d], g->som.data()); });
        if (rc != PINK_B200_OK) return rc;
        g->map_has_som = true;
    }
    return PINK_B200_OK;
}

} // namespace

extern "C" {

int pink_b200_device_count(void)
{
    int n = 0, usable = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    for (int d = 0; d < n; ++d) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess && major == 10) ++usable;
    }
    return usable;
}

int pink_b200_host_alloc(void** out, uint64_t bytes)
{
    if (!out) return report_error(PINK_B200_EINVAL, "null argument");
    *out = nullptr;
    const cudaError_t e = cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocPortable);
    if (e != cudaSuccess) return report_error(PINK_B200_ECUDA, cudaGetErrorString(e));
    return PINK_B200_OK;
}

int pink_b200_host_free(void* p)
{
    if (!p) return PINK_B200_OK;
    const cudaError_t e = cudaFreeHost(p);
    if (e != cudaSuccess) return report_error(PINK_B200_ECUDA, cudaGetErrorString(e));
    return PINK_B200_OK;
}

int pink_b200_group_create(const pink_b200_config* cfg, const int32_t* devices, uint32_t n_devices, pink_b200_group** out)
{
    if (!cfg || !out) return report_error(PINK_B200_EINVAL, "null argument");
    *out = nullptr;
    pink_b200_group* g = new (std::nothrow) pink_b200_group();
    if (!g) return report_error(PINK_B200_EINVAL, "out of host memory");
    g->cfg = *cfg;
    if (devices && n_devices) {
        g->devices.assign(devices, devices + n_devices);
    } else {
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); n = 0; }
        for (int d = 0; d < n; ++d) {
            int major = 0;
            if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d) == cudaSuccess && major == 10)
                g->devices.push_back(d);
        }
        if (n_devices && g->devices.size() > n_devices) g->devices.resize(n_devices);
    }
    if (g->devices.empty()) { delete g; return report_error(PINK_B200_ECUDA, "no sm_100 device is visible; this library has no other code path"); }
    // no more shards than neurons, and at most the ranks the peer exchange handles
    if (g->devices.size() > cfg->n_neurons) g->devices.resize(cfg->n_neurons);
    if (g->devices.size() > 16) g->devices.resize(16);
    // validate the configuration now (a throw-away context on the first device reports the reference's messages)
    pink_b200_config probe = *cfg;
    probe.device = g->devices[0]; probe.rank = 0; probe.world_size = 1;
    pink_b200_ctx* c = nullptr;
    const int rc = pink_b200_create(&probe, &c);
    if (rc != PINK_B200_OK) { delete g; return rc; }
    if (g->devices.size() == 1) { g->train.assign(1, c); }     // one device: this is the context of both roles
    else pink_b200_destroy(c);
    *out = g;
    return PINK_B200_OK;
}

int pink_b200_group_destroy(pink_b200_group* g)
{
    if (!g) return PINK_B200_OK;
    for (pink_b200_ctx* c : g->map) pink_b200_destroy(c);
    // the shards reference each other's memory: let every device finish before any context goes away
    for (pink_b200_ctx* c : g->train) if (c) pink_b200_synchronize(c);
    for (pink_b200_ctx* c : g->train) pink_b200_destroy(c);
    delete g;
    return PINK_B200_OK;
}

uint32_t pink_b200_group_size(const pink_b200_group* g) { return g ? (uint32_t)g->devices.size() : 0; }

int pink_b200_group_set_option(pink_b200_group* g, const char* name, long long value)
{
    if (!g || !name) return report_error(PINK_B200_EINVAL, "null argument");
    if (g->have_som || g->have_factors) return report_error(PINK_B200_ESTATE, "options must be set before the map and the factors");
    g->options.emplace_back(name, value);
    if (g->devices.size() == 1 && !g->train.empty()) return pink_b200_set_option(g->train[0], name, value);
    return PINK_B200_OK;
}

int pink_b200_group_set_som(pink_b200_group* g, const float* host_som)
{
    if (!g || !host_som) return report_error(PINK_B200_EINVAL, "null argument");
    const size_t n = (size_t)g->cfg.n_neurons * g->cfg.channels * g->cfg.neuron_dim * g->cfg.neuron_dim;
    g->som.assign(host_som, host_som + n);
    g->have_som = true;
    g->som_stale = false;
    g->train_has_som = g->map_has_som = false;
    if (!g->train.empty()) return ensure_train(g);
    return PINK_B200_OK;
}

int pink_b200_group_get_som(pink_b200_group* g, float* host_som)
{
    if (!g || !host_som) return report_error(PINK_B200_EINVAL, "null argument");
    if (!g->have_som) return report_error(PINK_B200_ESTATE, "pink_b200_group_set_som must be called first");
    const int rc = refresh_som(g);
    if (rc != PINK_B200_OK) return rc;
    std::copy(g->som.begin(), g->som.end(), host_som);
    return PINK_B200_OK;
}

int pink_b200_group_set_update_factors(pink_b200_group* g, const float* host_factors)
{
    if (!g || !host_factors) return report_error(PINK_B200_EINVAL, "null argument");
    const size_t n = (size_t)g->cfg.n_neurons * g->cfg.n_neurons;
    g->factors.assign(host_factors, host_factors + n);
    g->lut_layout[0] = ~0u;
    g->have_factors = true;
    g->train_has_factors = false;
    if (!g->train.empty()) return ensure_train(g);
    return PINK_B200_OK;
}

int pink_b200_group_set_update_lut(pink_b200_group* g, uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                   const float* host_lut, uint32_t n_classes)
{
    if (!g || !host_lut) return report_error(PINK_B200_EINVAL, "null argument");
    if (pink_b200_distance_classes(som_layout, dim0, dim1, dim2, nullptr, 0) != n_classes || n_classes == 0)
        return report_error(PINK_B200_EINVAL, "the table does not have one entry per distance class of this SOM layout");
    g->factors.assign(host_lut, host_lut + n_classes);
    g->lut_layout[0] = som_layout; g->lut_layout[1] = dim0; g->lut_layout[2] = dim1; g->lut_layout[3] = dim2;
    g->have_factors = true;
    g->train_has_factors = false;
    if (!g->train.empty()) return ensure_train(g);
    return PINK_B200_OK;
}

int pink_b200_group_train(pink_b200_group* g, const float* host_images, uint64_t n)
{
    if (!g || (!host_images && n)) return report_error(PINK_B200_EINVAL, "null argument");
    if (!g->have_som) return report_error(PINK_B200_ESTATE, "pink_b200_group_set_som must be called before training");
    if (!g->have_factors) return report_error(PINK_B200_ESTATE, "pink_b200_group_set_update_factors must be called before training");
    int rc = ensure_train(g);
    if (rc != PINK_B200_OK) return rc;
    g->som_stale = true;
    // every shard sees every image; the shards meet on the device, image by image
    return for_each_device(g->train.size(), [&](size_t d) { return pink_b200_train(g->train[d], host_images, n); });
}

int pink_b200_group_get_update_counts(pink_b200_group* g, uint32_t* host_counts)
{
    if (!g || !host_counts) return report_error(PINK_B200_EINVAL, "null argument");
    const size_t N = g->cfg.n_neurons;
    std::fill(host_counts, host_counts + N, 0u);
    if (g->train.empty()) return PINK_B200_OK;
    std::vector<std::vector<uint32_t>> part(g->train.size(), std::vector<uint32_t>(N));
    int rc = for_each_device(g->train.size(), [&](size_t d) { return pink_b200_get_update_counts(g->train[d], part[d].data()); });
    if (rc != PINK_B200_OK) return rc;
    for (const auto& p : part)
        for (size_t i = 0; i < N; ++i) host_counts[i] += p[i];      // each shard counts the hits of its own neurons
    return PINK_B200_OK;
}

int pink_b200_group_synchronize(pink_b200_group* g)
{
    if (!g) return report_error(PINK_B200_EINVAL, "null argument");
    if (g->train.empty()) return PINK_B200_OK;
    return for_each_device(g->train.size(), [&](size_t d) { return pink_b200_synchronize(g->train[d]); });
}

int pink_b200_group_map(pink_b200_group* g, const float* host_images, uint64_t n, float* host_dist, uint32_t* host_rot)
{
    if (!g || ((!host_images || !host_dist || !host_rot) && n)) return report_error(PINK_B200_EINVAL, "null argument");
    if (!g->have_som) return report_error(PINK_B200_ESTATE, "pink_b200_group_set_som must be called before mapping");
    // one device: its single context holds the whole map and serves both roles
    const bool single = g->devices.size() == 1;
    int rc = single ? ensure_train(g) : ensure_map(g);
    if (rc != PINK_B200_OK) return rc;
    const std::vector<pink_b200_ctx*>& ctx = single ? g->train : g->map;
    const size_t W = ctx.size(), N = g->cfg.n_neurons;
    const size_t isz = (size_t)g->cfg.channels * g->cfg.image_dim * g->cfg.image_dim;
    // contiguous ranges of images, as equal as possible; every range writes its own rows of the results
    return for_each_device(W, [&](size_t d) {
        const uint64_t lo = n * d / W, hi = n * (d + 1) / W;
        if (hi == lo) return (int)PINK_B200_OK;
        return pink_b200_map(ctx[d], host_images + lo * isz, hi - lo, host_dist + lo * N, host_rot + lo * N);
    });
}

} // extern "C"
