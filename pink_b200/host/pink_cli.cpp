// Command line front end with the options and file formats of the reference's `Pink`
// executable (src/Pink/main.cpp, src/Pink/main_generic.h:42-203,
// src/UtilitiesLib/InputData.cpp:83-495), driving the GPU library through its C ABI.
//
// Differences that follow from the library: images reach the GPU in batches (a reader
// thread fills one pinned-size host buffer while the previous one trains; the order of the
// images is exactly the reference's, shuffled or not), --cuda-off and
// --interpolation nearest_neighbor are refused (there is no CPU path and the reference's GPU
// path has no nearest-neighbour kernel either), --numthreads and --b1 are accepted and ignored.
// Two additions for scripting, which touch no GPU:  --inspect <file>  prints the header of a
// data, SOM, mapping or rotation file;  --dump-order <entries> <seed> <passes>  prints the
// order in which training presents the entries.
#include "../../include/pink_b200.h"
#include "pink_files.hpp"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <getopt.h>
#include <iostream>
#include <memory>
#include <thread>

using namespace pinkhost;

namespace {

struct Options
{
    bool verbose = false, use_flip = true, shuffle = true, write_rot_flip = false;
    uint32_t som_width = 10, som_height = 10, som_depth = 1, neuron_dim = 0, ed_dim = 0;
    uint32_t layout = PINK_B200_LAYOUT_CARTESIAN, seed = 1234, rotations = 360, iterations = 1;
    int progress_prints = 10;
    enum Init { ZERO, RANDOM, RANDOM_WITH_PREFERRED_DIRECTION, FILEINIT } init = ZERO;
    enum Path { UNDEFINED, TRAIN, MAP } path = UNDEFINED;
    enum Store { OFF, OVERWRITE, KEEP } inter_store = OFF;
    uint32_t func = PINK_B200_FUNC_GAUSSIAN;
    float sigma = 1.1f, damping = 0.2f, max_update_distance = -1.0f;
    uint32_t dist_type = PINK_B200_UINT8, ed_shape = PINK_B200_QUADRATIC;
    std::string data_file, result_file, som_file, rot_flip_file;
};

std::string upper(std::string s)
{
    for (char& c : s) c = (char)std::toupper((unsigned char)c);
    return s;
}

uint32_t to_u32(const char* s)
{
    const int v = std::stoi(s);
    if (v < 0) throw std::runtime_error("str_to_uint32_t: integer must be positive");
    return (uint32_t)v;
}

void usage()
{
    std::puts(
        "\n  Usage:\n\n"
        "    Pink [Options] --train <image-file> <result-file>\n"
        "    Pink [Options] --map   <image-file> <result-file> <SOM-file>\n\n"
        "  Options:\n\n"
        "    --dist-func, -f <string>             Distribution function for SOM update (see below).\n"
        "    --euclidean-distance-dimension, -e <int>  Dimension for euclidean distance calculation.\n"
        "    --euclidean-distance-shape <string>  Shape of euclidean distance region (quadratic = default, circular).\n"
        "    --euclidean-distance-type <string>   Data type for euclidean distance (float, uint16, uint8 = default).\n"
        "    --flip-off                           Switch off usage of mirrored images.\n"
        "    --help, -h                           Print this lines.\n"
        "    --init, -x <string>                  zero = default, random, random_with_preferred_direction, or SOM file.\n"
        "    --input-shuffle-off                  Switch off random shuffle of data input.\n"
        "    --inter-store <string>               Store intermediate SOM results (off = default, overwrite, keep).\n"
        "    --layout, -l <string>                Layout of SOM (cartesian = default, hexagonal).\n"
        "    --max-update-distance <float>        Maximum distance for SOM update (default = off).\n"
        "    --neuron-dimension, -d <int>         Dimension for quadratic SOM neurons (default = 2 * image-dimension / sqrt(2)).\n"
        "    --numrot, -n <int>                   Number of rotations (1 or a multiple of 4, default = 360).\n"
        "    --num-iter <int>                     Number of iterations (default = 1).\n"
        "    --progress, -p <int>                 Maximal number of progress information prints (default = 10).\n"
        "    --seed, -s <int>                     Seed for random number generator (default = 1234).\n"
        "    --store-rot-flip <string>            Store the rotation and flip information of the best match (mapping).\n"
        "    --som-width, --som-height, --som-depth <int>  Dimensions of the SOM (default = 10, 10, 1).\n"
        "    --verbose                            Print more output.\n"
        "    --version, -v                        Print version number.\n"
        "    --inspect <file>                     Print the header of a PINK binary file (no GPU needed).\n"
        "    --dump-order <entries> <seed> <passes>  Print the order of the training entries (no GPU needed).\n\n"
        "  Distribution function string:\n\n"
        "    <string> <float> <float>\n\n"
        "    gaussian sigma damping\n"
        "    unitygaussian sigma damping\n"
        "    mexicanhat sigma damping\n");
}

void check(int rc)
{
    if (rc != PINK_B200_OK) throw std::runtime_error(pink_b200_last_error());
}

int inspect(const std::string& path)
{
    std::ifstream is(path, std::ios::binary);
    if (!is) throw std::runtime_error("Error opening " + path);
    const std::string header = read_text_header(is);
    const int version = read_int(is), type = read_int(is);
    std::printf("{\"version\": %d, \"file_type\": %d, \"text_header_bytes\": %zu", version, type, header.size());
    auto dims = [&](const char* name) {
        (void)read_int(is);                                   // layout index
        const int n = read_int(is);
        std::printf(", \"%s\": [", name);
        for (int i = 0; i < n; ++i) std::printf("%s%d", i ? ", " : "", read_int(is));
        std::printf("]");
    };
    auto field = [&](const char* name) { const int v = read_int(is); std::printf(", \"%s\": %d", name, v); };
    if (type == 0) { field("data_type"); field("entries"); dims("dims"); }
    else if (type == 1) { field("data_type"); dims("som_dims"); dims("neuron_dims"); }
    else if (type == 2) { field("data_type"); field("entries"); dims("som_dims"); }
    else if (type == 3) { field("entries"); dims("som_dims"); }
    std::printf(", \"data_offset\": %lld}\n", (long long)is.tellg());
    return 0;
}

Options parse(int argc, char** argv)
{
    Options o;
    static const option longopts[] = {
        {"neuron-dimension", 1, nullptr, 'd'}, {"euclidean-distance-dimension", 1, nullptr, 'e'}, {"layout", 1, nullptr, 'l'},
        {"seed", 1, nullptr, 's'}, {"numrot", 1, nullptr, 'n'}, {"numthreads", 1, nullptr, 't'}, {"init", 1, nullptr, 'x'},
        {"progress", 1, nullptr, 'p'}, {"version", 0, nullptr, 'v'}, {"help", 0, nullptr, 'h'}, {"dist-func", 1, nullptr, 'f'},
        {"som-width", 1, nullptr, 0}, {"num-iter", 1, nullptr, 1}, {"flip-off", 0, nullptr, 2}, {"cuda-off", 0, nullptr, 3},
        {"verbose", 0, nullptr, 4}, {"interpolation", 1, nullptr, 5}, {"train", 1, nullptr, 6}, {"map", 1, nullptr, 7},
        {"inter-store", 1, nullptr, 8}, {"b1", 1, nullptr, 9}, {"max-update-distance", 1, nullptr, 10},
        {"som-height", 1, nullptr, 12}, {"som-depth", 1, nullptr, 13}, {"pbc", 0, nullptr, 14},
        {"store-rot-flip", 1, nullptr, 15}, {"euclidean-distance-type", 1, nullptr, 16},
        {"input-shuffle-off", 0, nullptr, 17}, {"euclidean-distance-shape", 1, nullptr, 18},
        {"inspect", 1, nullptr, 19}, {"dump-order", 1, nullptr, 20}, {nullptr, 0, nullptr, 0}};
    // the file arguments of --train / --map and the numbers of --dist-func follow their option as plain words
    auto word = [&](int index, const char* what) -> const char* {
        if (index >= argc || argv[index][0] == '-') throw std::runtime_error(std::string("Missing arguments for ") + what + " option.");
        return argv[index];
    };
    int c, idx = 0;
    while ((c = getopt_long(argc, argv, "vd:l:s:n:t:x:p:a:hf:e:", longopts, &idx)) != -1) {
        switch (c) {
            case 'd': o.neuron_dim = to_u32(optarg); break;
            case 'e': o.ed_dim = to_u32(optarg); break;
            case 0: o.som_width = to_u32(optarg); break;
            case 12: o.som_height = to_u32(optarg); break;
            case 13: o.som_depth = to_u32(optarg); break;
            case 1:
                o.iterations = to_u32(optarg);
                if (o.iterations == 0) throw std::runtime_error("Number of iterations must be larger than 0");
                break;
            case 'l': {
                const std::string s = upper(optarg);
                if (s == "CARTESIAN") o.layout = PINK_B200_LAYOUT_CARTESIAN;
                else if (s == "HEXAGONAL") o.layout = PINK_B200_LAYOUT_HEXAGONAL;
                else throw std::runtime_error("Unknown layout option " + s);
                break;
            }
            case 's': o.seed = to_u32(optarg); break;
            case 'p': o.progress_prints = std::atoi(optarg); break;
            case 'n':
                o.rotations = to_u32(optarg);
                if (o.rotations == 0 || (o.rotations != 1 && o.rotations % 4))
                    throw std::runtime_error("Number of rotations must be 1 or a multiple of 4");
                break;
            case 't': case 9: break;                           // host threads / CUDA block size: nothing to set here
            case 'x': {
                const std::string s = upper(optarg);
                if (s == "ZERO") o.init = Options::ZERO;
                else if (s == "RANDOM") o.init = Options::RANDOM;
                else if (s == "RANDOM_WITH_PREFERRED_DIRECTION") o.init = Options::RANDOM_WITH_PREFERRED_DIRECTION;
                else { o.init = Options::FILEINIT; o.som_file = optarg; }
                break;
            }
            case 2: o.use_flip = false; break;
            case 3: throw std::runtime_error("--cuda-off: this program has no CPU path");
            case 4: o.verbose = true; break;
            case 5: {
                const std::string s = upper(optarg);
                if (s == "NEAREST_NEIGHBOR") throw std::runtime_error("generate_rotated_images: unknown interpolation type");
                if (s != "BILINEAR") throw std::runtime_error("Unknown interpolation option " + s);
                break;
            }
            case 6: {
                o.path = Options::TRAIN;
                int i = optind - 1;
                o.data_file = word(i++, "--train");
                o.result_file = word(i++, "--train");
                optind = i;
                break;
            }
            case 7: {
                o.path = Options::MAP;
                int i = optind - 1;
                o.data_file = word(i++, "--map");
                o.result_file = word(i++, "--map");
                o.som_file = word(i++, "--map");
                optind = i;
                break;
            }
            case 8: {
                const std::string s = upper(optarg);
                if (s == "OFF") o.inter_store = Options::OFF;
                else if (s == "OVERWRITE") o.inter_store = Options::OVERWRITE;
                else if (s == "KEEP") o.inter_store = Options::KEEP;
                else throw std::runtime_error("Unknown intermediate storage option " + s);
                break;
            }
            case 10:
                o.max_update_distance = std::strtof(optarg, nullptr);
                if (o.max_update_distance <= 0.0f) throw std::runtime_error("max-update-distance must be positive.");
                break;
            case 14: throw std::runtime_error("Periodic boundary conditions are not supported in version 2.");
            case 15: o.write_rot_flip = true; o.rot_flip_file = optarg; break;
            case 16: {
                const std::string s = upper(optarg);
                if (s == "FLOAT") o.dist_type = PINK_B200_FLOAT;
                else if (s == "UINT16") o.dist_type = PINK_B200_UINT16;
                else if (s == "UINT8") o.dist_type = PINK_B200_UINT8;
                else throw std::runtime_error("Unknown euclidean distance type " + s);
                break;
            }
            case 17: o.shuffle = false; break;
            case 18: {
                const std::string s = upper(optarg);
                if (s == "QUADRATIC") o.ed_shape = PINK_B200_QUADRATIC;
                else if (s == "CIRCULAR") o.ed_shape = PINK_B200_CIRCULAR;
                else throw std::runtime_error("Unknown euclidean distance shape " + s);
                break;
            }
            case 19: std::exit(inspect(optarg));
            case 20: {
                int i = optind - 1;
                const uint32_t n = to_u32(word(i++, "--dump-order")), seed = to_u32(word(i++, "--dump-order"));
                const uint32_t passes = to_u32(word(i++, "--dump-order"));
                for (uint32_t p = 0; p < passes; ++p) {
                    const auto order = entry_order(n, (uint64_t)seed + p, true);
                    for (size_t k = 0; k < order.size(); ++k) std::printf("%s%u", k ? " " : "", order[k]);
                    std::printf("\n");
                }
                std::exit(0);
            }
            case 'v': std::printf("%s\n", pink_b200_version()); std::exit(0);
            case 'h': usage(); std::exit(0);
            case 'f': {
                const std::string s = upper(optarg);
                if (s == "GAUSSIAN") o.func = PINK_B200_FUNC_GAUSSIAN;
                else if (s == "UNITYGAUSSIAN") o.func = PINK_B200_FUNC_UNITY_GAUSSIAN;
                else if (s == "MEXICANHAT") o.func = PINK_B200_FUNC_MEXICAN_HAT;
                else throw std::runtime_error("Unknown distribution function " + s);
                int i = optind;
                o.sigma = std::strtof(word(i++, "--dist-func"), nullptr);
                o.damping = std::strtof(word(i++, "--dist-func"), nullptr);
                optind = i;
                break;
            }
            default: usage(); throw std::runtime_error("Unknown option");
        }
    }
    if (o.path == Options::MAP) o.init = Options::FILEINIT;
    else if (o.path == Options::UNDEFINED) { usage(); throw std::runtime_error("Unknown execution path."); }
    if (o.layout == PINK_B200_LAYOUT_HEXAGONAL) {
        if ((o.som_width - 1) % 2) throw std::runtime_error("For hexagonal layout only odd dimension supported.");
        if (o.som_width != o.som_height) throw std::runtime_error("For hexagonal layout som-width must be equal to som-height.");
        if (o.som_depth != 1) throw std::runtime_error("For hexagonal layout som-depth must be equal to 1.");
    }
    if (o.som_width < 2) throw std::runtime_error("som-width must be > 1.");
    if (o.som_height < 1) throw std::runtime_error("som-height must be > 0.");
    if (o.som_depth < 1) throw std::runtime_error("som-depth must be > 0.");
    if (o.som_depth > 1 && o.som_height < 2) throw std::runtime_error("som-depth > 1 needs som-height > 1.");
    return o;
}

// Reads entries order[first .. first + count) into dst.
void load_entries(std::ifstream& is, const DataFile& f, const std::vector<uint32_t>& order, size_t first, size_t count, float* dst)
{
    for (size_t k = 0; k < count; ++k) read_entry(is, f, order[first + k], dst + k * f.entry_floats);
}

struct Progress
{
    uint64_t total, section, next;
    std::chrono::steady_clock::time_point start = std::chrono::steady_clock::now();
    Progress(uint64_t total_, int prints) : total(total_)
    {
        const uint64_t p = std::max<uint64_t>(1, std::min<uint64_t>(total, (uint64_t)std::max(prints, 1)));
        section = total / p;
        next = section + (total % p ? 1 : 0);
    }
    void advance(uint64_t done)                                // `done` images finished so far
    {
        while (next <= done && next <= total) {
            const double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
            const int width = 70, pos = (int)(width * next / total);
            std::string bar(width, ' ');
            for (int i = 0; i < width; ++i) bar[i] = i < pos ? '=' : (i == pos ? '>' : ' ');
            std::printf("[%s] %d %% %.3f s\n", bar.c_str(), (int)(100.0 * next / total), s);
            next += section ? section : 1;
        }
        std::fflush(stdout);
    }
};

// Page-locked host array (pink_b200_host_alloc); falls back to nothing: allocation failure is an error.
template <typename T>
class PinnedBuffer
{
public:
    explicit PinnedBuffer(size_t n) : n_(n)
    {
        void* p = nullptr;
        check(pink_b200_host_alloc(&p, (uint64_t)n * sizeof(T)));
        p_ = static_cast<T*>(p);
    }
    PinnedBuffer(PinnedBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; }
    PinnedBuffer(const PinnedBuffer&) = delete;
    PinnedBuffer& operator=(const PinnedBuffer&) = delete;
    ~PinnedBuffer() { pink_b200_host_free(p_); }
    T* data() { return p_; }
    T& operator[](size_t i) { return p_[i]; }
    size_t size() const { return n_; }
private:
    T* p_ = nullptr;
    size_t n_ = 0;
};

int run(const Options& o)
{
    std::ifstream ifs(o.data_file, std::ios::binary);
    if (!ifs) throw std::runtime_error("Error opening " + o.data_file);
    const DataFile data = open_data_file(ifs);
    if (data.dims.size() < 2 || data.dims[data.dims.size() - 1] != data.dims[data.dims.size() - 2])
        throw std::runtime_error("Images must be quadratic.");
    const uint32_t image_dim = data.side(), channels = data.channels();

    // defaults derived from the image size (src/UtilitiesLib/InputData.cpp:452-478)
    uint32_t neuron_dim = o.neuron_dim, ed_dim = o.ed_dim;
    if (neuron_dim == 0) {
        neuron_dim = image_dim;
        if (o.rotations != 1) neuron_dim = (uint32_t)(2 * image_dim / std::sqrt(2.0) + 1);
    }
    if (ed_dim == 0) {
        ed_dim = image_dim;
        if (o.rotations != 1 && o.ed_shape == PINK_B200_QUADRATIC) ed_dim = (uint32_t)(ed_dim * std::sqrt(2.0) / 2);
    }
    if (ed_dim > neuron_dim) throw std::runtime_error("euclidean distance dimension must be equal or smaller than neuron dimension.");

    const uint32_t n_neurons = pink_b200_som_size(o.layout, o.som_width, o.som_height) * o.som_depth;
    if (n_neurons == 0) throw std::runtime_error("the SOM has no neurons");
    std::vector<int> som_dims = {(int)o.som_width};
    if (o.som_height > 1 || o.layout == PINK_B200_LAYOUT_HEXAGONAL) som_dims.push_back((int)o.som_height);
    if (o.som_depth > 1) som_dims.push_back((int)o.som_depth);
    std::vector<int> neuron_dims;
    if (data.dims.size() == 3) neuron_dims.push_back((int)channels);
    neuron_dims.push_back((int)neuron_dim);
    neuron_dims.push_back((int)neuron_dim);
    const size_t neuron_size = (size_t)channels * neuron_dim * neuron_dim;

    // initial map (src/SelfOrganizingMapLib/SOM.h:71-98)
    std::vector<float> som((size_t)n_neurons * neuron_size, 0.0f);
    std::string som_text_header;
    if (o.init == Options::RANDOM || o.init == Options::RANDOM_WITH_PREFERRED_DIRECTION) {
        std::mt19937 rng(o.seed);
        std::uniform_real_distribution<float> dist(0.0);
        for (float& v : som) v = dist(rng);
        if (o.init == Options::RANDOM_WITH_PREFERRED_DIRECTION)
            for (uint32_t n = 0; n < n_neurons; ++n)
                for (uint32_t i = 0; i < neuron_dim; ++i)
                    som[(size_t)n * neuron_dim * neuron_dim + (size_t)i * neuron_dim + i] = 1.0f;   // the reference's index (one channel)
    } else if (o.init == Options::FILEINIT) {
        SomFile f = read_som_file(o.som_file);
        if (f.data.size() != som.size()) throw std::runtime_error(o.som_file + " does not match the SOM and neuron dimensions");
        som = std::move(f.data);
        som_text_header = f.text_header;
    }

    if (o.verbose)
        std::printf("  SOM %u neurons (%s), neuron %u x %u x %u, image %u x %u, distance region %u (%s), %u rotations%s, %d entries\n",
                    n_neurons, o.layout == PINK_B200_LAYOUT_HEXAGONAL ? "hexagonal" : "cartesian", channels, neuron_dim, neuron_dim,
                    image_dim, image_dim, ed_dim, o.ed_shape == PINK_B200_CIRCULAR ? "circular" : "quadratic", o.rotations,
                    o.use_flip ? " + flip" : "", data.entries);

    pink_b200_config cfg{};
    cfg.n_neurons = n_neurons; cfg.channels = channels; cfg.image_dim = image_dim; cfg.neuron_dim = neuron_dim;
    cfg.ed_dim = ed_dim; cfg.ed_shape = o.ed_shape; cfg.n_rotations = o.rotations; cfg.use_flip = o.use_flip;
    cfg.dist_type = o.dist_type; cfg.interpolation = PINK_B200_BILINEAR; cfg.device = 0; cfg.rank = 0; cfg.world_size = 1;
    // every visible GPU takes part, as in the reference (src/CudaLib/CudaLib.cu:56-76): training shards the neurons
    // over them, mapping the images
    pink_b200_group* raw = nullptr;
    check(pink_b200_group_create(&cfg, nullptr, 0, &raw));
    std::unique_ptr<pink_b200_group, int (*)(pink_b200_group*)> ctx(raw, pink_b200_group_destroy);
    const uint32_t n_gpus = pink_b200_group_size(ctx.get());
    if (o.verbose) std::printf("  GPUs in use: %u\n", n_gpus);
    check(pink_b200_group_set_som(ctx.get(), som.data()));

    // images per host buffer; mapping deals a buffer over the GPUs, so it grows with their number
    const size_t batch = o.path == Options::TRAIN ? 256 : 256 * (size_t)n_gpus;
    // page-locked staging: the copies to the devices run asynchronously while the reader thread fills the other buffer
    PinnedBuffer<float> buffers[2] = {PinnedBuffer<float>(batch * data.entry_floats), PinnedBuffer<float>(batch * data.entry_floats)};
    const uint32_t entries = (uint32_t)data.entries;

    if (o.path == Options::TRAIN) {
        // one update factor per distinct map distance of the grid (the reference fills an N x N table, Trainer.h:69-76)
        const uint32_t depth = o.som_depth > 1 ? o.som_depth : 1;
        const uint32_t classes = pink_b200_distance_classes(o.layout, o.som_width, o.som_height, depth, nullptr, 0);
        if (classes == 0) throw std::runtime_error("unsupported SOM layout");
        std::vector<float> factors(classes);
        check(pink_b200_update_lut(o.layout, o.som_width, o.som_height, depth, o.func, o.sigma, o.damping,
                                   o.max_update_distance, factors.data(), classes));
        check(pink_b200_group_set_update_lut(ctx.get(), o.layout, o.som_width, o.som_height, depth, factors.data(), classes));
        const uint64_t total = (uint64_t)entries * o.iterations;
        Progress progress(total, o.progress_prints);
        std::vector<uint64_t> stores;
        if (o.inter_store != Options::OFF) stores = report_points(total, o.progress_prints);
        size_t store_idx = 0, keep_count = 0;
        uint64_t done = 0;
        auto store_map = [&](const std::string& path) {
            check(pink_b200_group_get_som(ctx.get(), som.data()));
            write_som_file(path, som_text_header, som_dims, neuron_dims, som.data(), som.size());
        };
        for (uint32_t it = 0; it < o.iterations; ++it) {
            // the seed changes with every pass so that every pass has its own order (main_generic.h:83-86)
            const std::vector<uint32_t> order = entry_order(entries, (uint64_t)o.seed + it, o.shuffle);
            // chunks end at the images after which an intermediate map is due
            std::vector<std::pair<size_t, size_t>> chunks;    // (first, count) within this pass
            for (size_t first = 0; first < entries;) {
                size_t count = std::min<size_t>(batch, entries - first);
                const uint64_t global_first = (uint64_t)it * entries + first;
                for (size_t s = store_idx; s < stores.size(); ++s) {
                    const uint64_t at = stores[s];            // global index of the image to store after
                    if (at < global_first) continue;
                    if (at < global_first + count) count = (size_t)(at - global_first) + 1;
                    break;
                }
                chunks.push_back({first, count});
                first += count;
            }
            std::ifstream reader_stream(o.data_file, std::ios::binary);
            std::thread reader;
            if (!chunks.empty()) load_entries(reader_stream, data, order, chunks[0].first, chunks[0].second, buffers[0].data());
            for (size_t k = 0; k < chunks.size(); ++k) {
                if (k + 1 < chunks.size())
                    reader = std::thread(load_entries, std::ref(reader_stream), std::cref(data), std::cref(order), chunks[k + 1].first,
                                         chunks[k + 1].second, buffers[(k + 1) & 1].data());
                check(pink_b200_group_train(ctx.get(), buffers[k & 1].data(), chunks[k].second));
                check(pink_b200_group_synchronize(ctx.get()));      // the reader thread refills this buffer next
                done += chunks[k].second;
                if (reader.joinable()) reader.join();
                progress.advance(done);
                while (store_idx < stores.size() && stores[store_idx] + 1 == done) {
                    std::string name = o.result_file;
                    if (o.inter_store == Options::KEEP) {
                        const size_t dot = name.find_last_of('.');
                        name.insert(dot == std::string::npos ? name.size() : dot, "_" + std::to_string(keep_count++));
                    }
                    if (o.verbose) std::printf("  Write intermediate SOM to %s ... ", name.c_str());
                    store_map(name);
                    if (o.verbose) std::printf("done.\n");
                    ++store_idx;
                }
            }
        }
        std::printf("  Write final SOM to %s ... ", o.result_file.c_str());
        store_map(o.result_file);
        std::printf("done.\n");
        if (o.verbose) {
            std::vector<uint32_t> counts(n_neurons);
            check(pink_b200_group_get_update_counts(ctx.get(), counts.data()));
            std::printf("\n  Number of updates of each neuron:\n\n");
            for (uint32_t i = 0; i < n_neurons; ++i) std::printf("%u%s", counts[i], (i + 1) % o.som_width ? " " : "\n");
            std::printf("\n");
        }
    } else {
        std::ofstream result(o.result_file, std::ios::binary);
        if (!result) throw std::runtime_error("Error opening " + o.result_file);
        write_mapping_header(result, data.entries, som_dims);
        std::ofstream rot_flip;
        if (o.write_rot_flip) {
            rot_flip.open(o.rot_flip_file, std::ios::binary);
            if (!rot_flip) throw std::runtime_error("Error opening " + o.rot_flip_file);
            write_rot_flip_header(rot_flip, data.entries, som_dims);
        }
        std::vector<uint32_t> order(entries);
        std::iota(order.begin(), order.end(), 0u);
        PinnedBuffer<float> dist(batch * n_neurons);
        PinnedBuffer<uint32_t> rot(batch * n_neurons);
        Progress progress(entries, o.progress_prints);
        const float angle_step = static_cast<float>(2.0 * M_PI) / o.rotations;
        std::ifstream reader_stream(o.data_file, std::ios::binary);
        std::thread reader;
        load_entries(reader_stream, data, order, 0, std::min<size_t>(batch, entries), buffers[0].data());
        for (size_t first = 0, k = 0; first < entries; first += batch, ++k) {
            const size_t count = std::min<size_t>(batch, entries - first);
            if (first + count < entries)
                reader = std::thread(load_entries, std::ref(reader_stream), std::cref(data), std::cref(order), first + count,
                                     std::min<size_t>(batch, entries - first - count), buffers[(k + 1) & 1].data());
            check(pink_b200_group_map(ctx.get(), buffers[k & 1].data(), count, dist.data(), rot.data()));
            result.write(reinterpret_cast<const char*>(dist.data()), (std::streamsize)(count * n_neurons * sizeof(float)));
            if (o.write_rot_flip) {
                for (size_t i = 0; i < count * n_neurons; ++i) {
                    const char flip = (char)(rot[i] / o.rotations);
                    const float angle = (rot[i] % o.rotations) * angle_step;
                    rot_flip.write(&flip, 1);
                    rot_flip.write(reinterpret_cast<const char*>(&angle), sizeof(float));
                }
            }
            if (reader.joinable()) reader.join();
            progress.advance(first + count);
        }
    }
    return 0;
}

} // namespace

int main(int argc, char** argv)
{
    try {
        return run(parse(argc, argv));
    } catch (std::exception const& e) {
        std::fprintf(stderr, "PINK exception: %s\n", e.what());
        return 1;
    }
}
