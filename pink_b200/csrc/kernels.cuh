// Shared declarations of the hot-path kernels: geometry of one SOM/image
// configuration, device-side operand layout, and the host launchers the C-ABI
// layer calls.  Notation (as in the PINK sources): N neurons, R rotations,
// T = R * (flip ? 2 : 1) transforms, C channels, nd neuron side, id image
// side, ed side of the distance region, P = C*nd*nd, K = C*ed*ed.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <functional>

struct pink_b200_config;

namespace pinkb {

// Distance modes; numbering follows pink::DataType (UtilitiesLib/DataType.h).
enum : int { kModeF32 = 0, kModeU16 = 1, kModeU8 = 2 };
constexpr int kModeTf32 = 3;      // internal: the tensor-core filter pass of float32 mapping (never a Geometry::mode)

// Status codes a kernel may leave in the device status word.
enum : int { kDevOk = 0, kDevTimeoutProducer = 1, kDevTimeoutMma = 2, kDevTimeoutEpilogue = 3,
             kDevTimeoutUpdateProducer = 11, kDevTimeoutUpdateConsumer = 12, kDevTimeoutExchange = 13, kDevTimeoutRotation = 14,
             kDevTimeoutGrid = 15 };

struct Geometry
{
    uint32_t C, id, nd, ed;     // channels, image side, neuron side, distance-region side
    uint32_t R, T, q;           // rotations, transforms, rotations per quadrant (R/4, 0 when R == 1)
    uint32_t flip;
    uint32_t off;               // crop offset uint32((nd - ed) * 0.5)
    uint32_t P, Pp;             // neuron size and its row stride in floats (multiple of 4)
    uint32_t K, Kp;             // distance length and operand row stride in ELEMENTS:
                                //   integer modes: multiple of 128 (bytes per plane row)
                                //   float mode:    multiple of 16 floats
    int mode;
    // Circular distance region (src/ImageProcessingLib/circular_euclidean_distance.h:36-60): device table of
    // ed entries {first column, end column} of each region row, in region-local columns; null = the whole
    // ed x ed square.  Operand elements outside the circle are written as zeros, which removes them from
    // every term of the distance.
    const ushort2* circle;
};

__device__ __forceinline__ bool in_region(const Geometry& g, uint32_t row, uint32_t col)
{
    if (!g.circle) return true;
    const ushort2 r = g.circle[row];
    return col >= r.x && col < r.y;
}

// Ordering code of a per-neuron minimum.  Integer modes: the exact integer sum
// S; float mode: the IEEE bit pattern of the non-negative float sum.  A key
// packs (code << kKeyShift) | transform so that an unsigned 64-bit minimum
// yields the smallest distance and, among equals, the lowest transform index
// (the reference's first-minimum rule).
__host__ __device__ constexpr uint32_t key_shift(int mode) { return mode == kModeU16 ? 16u : 32u; }
constexpr unsigned long long kKeyEmpty = ~0ull;

// Local-shard best-matching-unit record exchanged between ranks.
struct BmuPair { unsigned long long code; unsigned long long neuron; };

// ---- rotation set -----------------------------------------------------------
// images: [n_img][C][id][id] float.  cs/sn: [q] cos/sin of t*2*pi/R (entry 0 unused).
// base_out (nullable): [n_img][max(q,1)][C][nd][nd] float base rotations.
// b0/b1: operand planes [n_img*T][Kp] (u8: b0; u16: b0 = high byte, b1 = low
// byte; f32: b0 as float, and -- when b1 is given -- b1 / b2 the two TF32 word
// planes of the mapping estimate: value with its low 13 mantissa bits cleared,
// and the rest).  bnorm: [n_img*T] sum of squares (u32 for u8, u64 for u16,
// float for f32 with planes, else unused for f32).
// rmax (nullable): [n_img] words zeroed by the caller; receives the bit pattern of max |pixel| over each image's base rotations.
cudaError_t launch_rotate(const Geometry& g, const float* images, uint32_t n_img, const float* cs, const float* sn,
                   float* base_out, void* b0, void* b1, void* bnorm, cudaStream_t st, uint32_t* rmax = nullptr,
                   void* b2 = nullptr);

// ---- SOM operand ------------------------------------------------------------
// som: [n][Pp] float.  a0/a1/anorm: as b0/b1/bnorm with one row per neuron.
// wrange (nullable): [n] bit patterns of {min |w|, max |w|} over each whole neuron.
cudaError_t launch_quantize_som(const Geometry& g, const float* som, uint32_t n, void* a0, void* a1, void* anorm,
                         cudaStream_t st, uint2* wrange = nullptr);

// ---- distances + minimum over transforms ------------------------------------
struct DistanceArgs
{
    const void* a0; const void* a1; const void* anorm; uint32_t n;          // SOM operand, n local neurons
    const void* b0; const void* b1; const void* bnorm; uint32_t n_img;      // transform operand
    unsigned long long* keys;   // [n_img][n], must hold kKeyEmpty on entry
    void* s_out;                // optional full matrix [n_img][n][T]: u32 (u8), u64 (u16), f32 (f32)
    int* status;                // device status word
    // Optional tail (one image, integer modes): the last block to finish reduces keys[0..n) to this
    // shard's record and publishes it as launch_bmu phase 1 would.  tail_counter: zeroed uint32.
    const struct BmuArgs* tail; uint32_t* tail_counter;
    uint32_t single_cta;        // 1: never pair blocks for one M = 256 MMA (diagnostic)
};
// True when launch_distance honours DistanceArgs::tail for this geometry.
bool distance_has_tail(const Geometry& g);
// Returns cudaSuccess or the launch / tensor-map error; *why receives a static message.
cudaError_t launch_distance(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why);

// float32 mapping as filter + exact pass (distance_tc.cu, filter_f32.cu).  launch_split_tf32 writes, for `rows`
// operand rows of Kp floats, the two TF32 word planes (hi = the value with its low 13 mantissa bits cleared,
// lo = value - hi, exact) and the float |row|^2.  launch_distance_tf32 fills est[n_img][n][T] with
// max(|a|^2 + |b|^2 - 2 (ah.bh + ah.bl + al.bh), 0).  launch_refine_f32 then, per (image, neuron), keeps every
// transform whose estimate could still be the minimum given the error bound eps * (|a|^2 + |b|^2) on both sides,
// computes those distances exactly from the float operands (direct differences) and stores the key
// (float bits << 32 | transform) of the first minimum; cand_count (nullable) accumulates the exact evaluations.
cudaError_t launch_split_tf32(const float* src, uint64_t rows, uint32_t Kp, float* hi, float* lo, float* norm, cudaStream_t st);
cudaError_t launch_distance_tf32(const Geometry& g, const DistanceArgs& a, cudaStream_t st, const char** why);
cudaError_t launch_refine_f32(const Geometry& g, const float* A, const float* anorm, uint32_t n, const float* B, const float* bnorm,
                              uint32_t n_img, const float* est, float eps, unsigned long long* keys,
                              unsigned long long* cand_count, cudaStream_t st);

// ---- update factors ----------------------------------------------------------------
// Either the N x N table of the reference (Trainer.h:69-76), this shard's columns of it, or -- for the grid layouts,
// where the map distance takes few distinct values -- one value per distance class: lut[class(coords[bmu], coords[n])].
struct FactorSource
{
    const float* table;         // [N_global][n_local], column = local neuron; null when the classes are used
    const short4* coords;       // [N_global] grid position of every neuron (cartesian: x, y, z; hexagonal: axial q, r)
    const float* lut;           // [classes]
    uint32_t hexagonal, dim0, dim1;
};

#ifdef __CUDACC__
__device__ __forceinline__ float factor_of(const FactorSource& fs, uint32_t bmu, uint32_t local, uint32_t global, uint32_t n_local)
{
    if (fs.table) return fs.table[(size_t)bmu * n_local + local];
    const short4 a = fs.coords[bmu], b = fs.coords[global];
    const int dx = a.x - b.x, dy = a.y - b.y, dz = a.z - b.z;
    uint32_t cls;
    if (fs.hexagonal) cls = ((dx >= 0) == (dy >= 0)) ? (uint32_t)abs(dx + dy) : (uint32_t)max(abs(dx), abs(dy));
    else cls = ((uint32_t)abs(dz) * fs.dim0 + (uint32_t)abs(dy)) * fs.dim1 + (uint32_t)abs(dx);
    return fs.lut[cls];
}
#endif

// ---- best matching unit and work list of the update ----------------------------
// One neuron the update must rewrite: local index, update factor, and its best
// transform decoded into the base rotation tq and the affine map
// src = c*nd*nd + ax*x + ay*y + a0 from a neuron pixel (x, y) to that base
// rotation (flip reverses rows last, src/CudaLib/flip_kernel.h:28; a quarter
// turn maps (x, y) <- (nd-1-y, x), src/CudaLib/rotate_90_degrees_list.h:28).
struct UpdateItem { uint32_t n, tq; int32_t ax, ay, a0; float f; };

// Exchange of the per-rank best-matching-unit records through peer memory: every rank owns
// kXchgSlots x world records; rank r writes its record of step `seq` into entry
// [seq % kXchgSlots][r] of EVERY rank's array with two plain 8-byte stores over NVLink, and the
// update kernel polls its own array.  Each word carries the low 8 bits of `seq` as a tag
// (w0 = code << 8 | tag, w1 = neuron << 8 | tag), so a word is valid as soon as its tag matches
// and no fence or flag has to follow the data; a slot is reused every kXchgSlots steps, whose
// tags differ.  A rank can be at most one step ahead of another (it needs the other's record to
// finish a step), so the ring is never overrun.  Codes stay below 2^56 (checked on the host).
struct XchgRecord { unsigned long long w0, w1; };
constexpr uint32_t kXchgSlots = 4;
constexpr uint32_t kXchgMaxRanks = 16;

struct BmuArgs
{
    unsigned long long* keys; uint32_t n, first_neuron, shift;   // this shard's per-neuron minima (re-armed in phase 2)
    uint32_t neuron_stride;           // local neuron j is global neuron first_neuron + j * neuron_stride
    BmuPair* pairs; uint32_t rank, world;                        // per-rank records (world entries)
    FactorSource factors;             // update factors of (best matching unit, neuron)
    UpdateItem* items; uint32_t* n_items;   // out: neurons with a non-zero factor, ascending, and their number
    uint32_t* counts;                 // [N_global] BMU hit counters (incremented by the owner)
    uint32_t* bmu_log;                // nullable: receives the global BMU index of this step
    uint32_t R, q, nd;                // geometry needed to decode a transform index
    uint32_t magic_R, magic_q;        // multiply-high reciprocals of R and q (0 = divisor 1); need T * R < 2^32
    uint32_t* arrive;                 // fused update only: block arrival counter, zero between launches
    unsigned long long* stats;        // nullable: [0] += neurons with a non-zero factor, [1] += neurons written back
    // peer-memory exchange (world > 1, xchg_seq != 0): this rank's record array and every rank's (own included)
    XchgRecord* xchg_local; XchgRecord* xchg_peer[kXchgMaxRanks]; unsigned long long xchg_seq;
    int* status;                      // device status word (receives a code if the wait for the records expires)
    unsigned long long xchg_timeout_ns;   // wall-clock limit of the wait for the other ranks' records (0: a second)
};
// phase bit 0: reduce keys[0..n) to this shard's (code, first_neuron + argmin) record in pairs[rank];
// phase bit 1: pick the global best matching unit from pairs, count the hit, re-arm the keys and emit
// the work list.  A single-GPU step runs both in one launch; with several ranks the exchange of the
// records sits between them.
cudaError_t launch_bmu(const BmuArgs& a, uint32_t phase, cudaStream_t st);

// ---- neighbourhood update ---------------------------------------------------
struct UpdateArgs
{
    float* som;                       // [n][Pp]
    const float* base;                // [max(q,1)][C][nd][nd] base rotations of the current image
    const UpdateItem* items; const uint32_t* n_items;   // work list from launch_bmu
    uint32_t n;                       // local neurons (upper bound of the work list)
    void* a0; void* a1; void* anorm;  // SOM operand rows to refresh
    // Fused form only (both nullable together): per-neuron {min |w|, max |w|} as float bit patterns,
    // kept up to date by the kernel, and the bit pattern of max |r| over the current image's base
    // rotations.  With them the kernel leaves out neurons that provably cannot change (see cannot_change).
    uint2* wrange; const uint32_t* rmax;
};

// True when  w - (w - r) * f  (each operation rounded to nearest, as the update computes it) returns w
// itself for EVERY w with wmin <= |w| <= wmax and every |r| <= rmax:  the product is at most
// up(up(wmax + rmax) * f) in magnitude, and anything below a quarter of the spacing of the floats at
// wmin rounds away in the final subtraction.  Zero, denormal or NaN inputs give no guarantee (false).
// Arguments are float bit patterns of non-negative values; f > 0.
__host__ __device__ inline bool cannot_change(float f, uint32_t wmin_bits, uint32_t wmax_bits, uint32_t rmax_bits)
{
#ifdef __CUDA_ARCH__
    if (wmin_bits < 0x00800000u || wmax_bits >= 0x7F800000u || rmax_bits >= 0x7F800000u) return false;
    const float quarter_ulp = __uint_as_float(wmin_bits & 0x7F800000u) * 2.98023224e-8f;      // 2^e * 2^-25, exact
    const float bound = __fmul_ru(__fadd_ru(__uint_as_float(wmax_bits), __uint_as_float(rmax_bits)), fabsf(f));
    return bound < quarter_ulp;
#else
    (void)f; (void)wmin_bits; (void)wmax_bits; (void)rmax_bits;
    return false;
#endif
}
// Unfused form: one block per neuron works through the list launch_bmu (phase 2) wrote.
cudaError_t launch_update(const Geometry& g, const UpdateArgs& a, cudaStream_t st, int* status);
// Fused form, a persistent pipelined kernel: it reduces the keys (world == 1) or the exchanged
// per-rank records (world > 1, after launch_bmu phase 1 and the exchange) to the best matching unit,
// counts the hit, derives its work list and re-arms the keys itself; a.items / a.n_items and
// launch_bmu phase 2 are not used.  Available when update_can_fuse(g); b.arrive must point to a
// zeroed counter.  status: device status word that receives a code if a bounded wait expires.
bool update_can_fuse(const Geometry& g);
cudaError_t launch_update_fused(const Geometry& g, const UpdateArgs& a, const BmuArgs& b, cudaStream_t st, int* status);

// ---- whole training steps of a batch of images in ONE persistent kernel (train_steps.cu) -------------
// One block per SM stays resident for the whole batch and walks image by image through the phases
// distance -> (grid barrier) -> best matching unit, work list, update -> (grid barrier), so that an
// image costs no kernel launch, no set-up and no host round trip.  Integer distance modes only.
constexpr uint32_t kStepBatchMax = 16;          // images per launch
constexpr uint32_t kStepMaxOwned = 32;          // neurons one block may own
constexpr uint32_t kStepStampWords = 12;        // opt-in timeline words per image and block

// Control words of one launch; the host sets every byte to 0xFF before the launch.
//   bmu_word[i]: minimum over all (neuron, transform tile) partial minima of image i of
//                (code << s) | global neuron index, s = 32 (uint8) or 16 (uint16)
//   bar:         arrival counter of the grid barriers (counts up from 0xFFFFFFFF, i.e. -1)
struct StepCtrl { unsigned long long bmu_word[kStepBatchMax]; uint32_t bar; uint32_t pad; };

// Launch shape and shared-memory layout, fixed per context.
struct StepPlan
{
    uint32_t pair;                       // blocks work as cta_group::2 pairs in the distance phase
    uint32_t grid;                       // blocks (all resident at once); even when pair
    uint32_t n_tile, n_tiles, m_units;   // transform tile width, tiles per image, neuron tiles (pairs of tiles when pair)
    uint32_t ring_stages, b_bytes;       // TMA ring of the distance phase
    uint32_t upd_stages, upd_stage_bytes, upd_off_base;     // stages of the update phase: {neuron plane, base rotation plane}
    uint32_t col_chunks, row_blocks, rows_per_block;        // consumer task grid per plane
    uint32_t owned_per_block;            // length of a block's row in the ownership table
    uint32_t smem_bytes;                 // dynamic shared memory
};

struct StepArgs
{
    uint32_t plain_launch;            // host only: launch without the cooperative attribute (profilers that refuse it)
    // distance phase
    void* a0; void* a1; void* anorm; uint32_t n;                       // SOM operand of this shard (rows are rewritten by the update phase)
    const void* b0; const void* b1; const void* bnorm; uint32_t b_rows; // transform operand buffer (all rows) and its row count
    uint32_t b_row0;                  // row of the first image's transform 0 in that buffer
    unsigned long long* keys;         // [n], kKeyEmpty on entry and on exit
    // update phase
    float* som;                       // [n][Pp]
    const float* base;                // base rotations of the first image; consecutive images follow
    uint2* wrange; const uint32_t* rmax;   // nullable together: value ranges (see cannot_change); rmax[i] for image i
    FactorSource factors;             // update factors of (best matching unit, neuron)
    const uint32_t* owners;           // [grid][owned_per_block] local neuron indices, ~0u = none
    // bookkeeping
    uint32_t n_img, first_neuron, neuron_stride, rank, world;   // local neuron j is global neuron first_neuron + j * neuron_stride
    uint32_t* counts; uint32_t* bmu_log; unsigned long long* stats; int* status;
    StepCtrl* ctrl;
    unsigned long long* stamps;       // nullable: [n_img][grid][kStepStampWords] device-timer stamps of every block (see train_steps.cu)
    // peer-memory exchange of the shards' records (world > 1): as in BmuArgs; the record of image i carries xchg_seq0 + i
    XchgRecord* xchg_local; XchgRecord* xchg_peer[kXchgMaxRanks]; unsigned long long xchg_seq0;
    unsigned long long xchg_timeout_ns;   // wall-clock limit of the wait for the other ranks' records
};

// Fills `plan` and returns true when the persistent kernel can run this geometry on the current device.
bool step_plan(const Geometry& g, uint32_t n_local, uint32_t n_global, StepPlan* plan, const char** why_not);
// Which block updates which neuron: owners[b * owned_per_block + j], balanced so that the neurons close to any
// best matching unit (large update factors) are spread over different blocks.
// closeness(i, m): update factor between global neurons i and m (any symmetric non-negative measure of nearness).
void step_assign_owners(const std::function<float(uint32_t, uint32_t)>& closeness, uint32_t first, uint32_t stride,
                        uint32_t count, const StepPlan& plan, uint32_t* owners);
cudaError_t launch_train_steps(const Geometry& g, const StepPlan& plan, const StepArgs& a, cudaStream_t st, const char** why);

// ---- mapping epilogue -------------------------------------------------------
// dist[i][n] = sqrt(reported distance), rot[i][n] = transform; re-arms the keys.
cudaError_t launch_map_finalize(const Geometry& g, unsigned long long* keys, uint32_t n_img, uint32_t n,
                         float* dist, uint32_t* rot, cudaStream_t st);

cudaError_t launch_fill_keys(unsigned long long* keys, size_t count, cudaStream_t st);

// ---- rotation sets computed in shares by the ranks (see rotshare.cu) -----------------------
// Stores `value` into entry `entry` of every rank's flag array (peer_flags[r], r < world <= kXchgMaxRanks).
cudaError_t launch_flag_publish(unsigned long long* const* peer_flags, uint32_t world, uint32_t entry,
                                unsigned long long value, cudaStream_t st);
// Waits (at most timeout_ns of wall clock; status receives kDevTimeoutRotation on expiry) until row[r] holds
// `value` for every r != self.
cudaError_t launch_flag_wait(const unsigned long long* row, uint32_t world, uint32_t self, unsigned long long value,
                             int* status, unsigned long long timeout_ns, cudaStream_t st);

// Helpers of the C-ABI layer that entry points defined beside their kernels use:
// validate a configuration into a Geometry (returns a PINK_B200_* status and sets
// the calling thread's error message), and record an error message.
int geometry_from_config(const pink_b200_config* cfg, Geometry* g);
int report_error(int code, const char* msg);

} // namespace pinkb
