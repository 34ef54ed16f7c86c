/*
 * pink_b200.h -- C ABI of the B200-native implementation of PINK's
 * rotation/flip-invariant SOM hot path (rotate/flip -> distance matrix ->
 * minimum over rotations -> best matching unit -> neighbourhood update, and
 * the mapping variant).
 *
 * The reference has no FFI layer for this path: its boundary is the C++
 * template specialisation Trainer<..., UseGPU=true> / Mapper<..., UseGPU=true>
 * (src/SelfOrganizingMapLib/Trainer.h:198-333, Mapper.h:126-229), which owns
 * device buffers and calls three CudaLib entry points that take
 * thrust::device_vector arguments.  The functions below are what a binding of
 * that boundary needs: plain pointers and sizes, an opaque context in place of
 * the Trainer/Mapper object's device state, and an int status in place of
 * exceptions and exit().  Each entry names the reference code it stands for.
 *
 * Conventions
 *   - every function returns PINK_B200_OK (0) or a negative PINK_B200_E* code;
 *     nothing throws, nothing calls exit().  pink_b200_last_error() returns a
 *     message for the calling thread's most recent failure.
 *   - "host" pointers are ordinary (pageable or pinned) host memory, "dev"
 *     pointers are device memory of the context's device.
 *   - images are float32 [C][id][id] (C == 1 for 2-D data), SOMs are float32
 *     [N][C][nd][nd], both row-major without padding.
 *   - a context is used from one host thread at a time.
 *   - there is no CPU fallback: every compute entry runs CUDA kernels and
 *     fails with PINK_B200_ECUDA where no sm_100 device is present.
 */
#ifndef PINK_B200_H
#define PINK_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PINK_B200_OK          0
#define PINK_B200_EINVAL     -1   /* bad argument or unsupported configuration      */
#define PINK_B200_ECUDA      -2   /* CUDA runtime / driver error                    */
#define PINK_B200_ENCCL      -3   /* NCCL error or NCCL library not loadable        */
#define PINK_B200_ETIMEOUT   -4   /* a bounded device-side wait expired             */
#define PINK_B200_ESTATE     -5   /* call not valid in the context's current state  */

/* Distance modes; numbering of pink::DataType (src/UtilitiesLib/DataType.h:17-22). */
#define PINK_B200_FLOAT   0
#define PINK_B200_UINT16  1
#define PINK_B200_UINT8   2

/* Shape of the distance region (src/UtilitiesLib/EuclideanDistanceShape.h:15-19). */
#define PINK_B200_QUADRATIC 0
#define PINK_B200_CIRCULAR  1

/* Interpolation (src/UtilitiesLib/Interpolation.h:15-19); only BILINEAR exists
 * on the reference's GPU path (src/CudaLib/generate_rotated_images.h:119-121). */
#define PINK_B200_NEAREST_NEIGHBOR 0
#define PINK_B200_BILINEAR         1

/* SOM grid layouts (src/UtilitiesLib/Layout.h:15-19). */
#define PINK_B200_LAYOUT_CARTESIAN 0
#define PINK_B200_LAYOUT_HEXAGONAL 1

/* Neighbourhood functions (src/UtilitiesLib/DistributionFunctor.h:32-104). */
#define PINK_B200_FUNC_GAUSSIAN        0   /* p0 = sigma, p1 = damping */
#define PINK_B200_FUNC_UNITY_GAUSSIAN  1   /* p0 = sigma, p1 = damping */
#define PINK_B200_FUNC_MEXICAN_HAT     2   /* p0 = sigma, p1 = damping */
#define PINK_B200_FUNC_STEP            3   /* p0 = value               */

typedef struct pink_b200_ctx pink_b200_ctx;

/* Everything the Trainer / Mapper constructors take that shapes device state
 * (src/SelfOrganizingMapLib/Trainer.h:211-215, Mapper.h:134-137). */
typedef struct pink_b200_config {
    uint32_t n_neurons;        /* N: neurons of the whole SOM                                  */
    uint32_t channels;         /* C: 1 for 2-D images, dimension 0 of 3-D images ("spacing")   */
    uint32_t image_dim;        /* id: images are square                                        */
    uint32_t neuron_dim;       /* nd                                                           */
    uint32_t ed_dim;           /* euclidean_distance_dim                                       */
    uint32_t ed_shape;         /* PINK_B200_QUADRATIC                                          */
    uint32_t n_rotations;      /* number_of_rotations: 1 or a multiple of 4                    */
    uint32_t use_flip;         /* 0 / 1                                                        */
    uint32_t dist_type;        /* PINK_B200_FLOAT / UINT16 / UINT8                             */
    uint32_t interpolation;    /* PINK_B200_BILINEAR                                           */
    int32_t  device;           /* CUDA device ordinal                                          */
    uint32_t rank;             /* this process's index among the neuron shards                 */
    uint32_t world_size;       /* number of neuron shards (1 = whole SOM on this device)       */
    uint32_t max_batch;        /* images staged per internal batch (0 = default)               */
} pink_b200_config;

/* Message of the calling thread's most recent failing call ("" if none). */
const char* pink_b200_last_error(void);

/* Library version string. */
const char* pink_b200_version(void);

/* ---- context life cycle ---------------------------------------------------- */

/* Validates the configuration (errors of TrainerCommon / MapperCommon,
 * src/SelfOrganizingMapLib/Trainer.h:66-67, Mapper.h:59-66, and "Images must
 * be quadratic" is implied by image_dim) and allocates the device state the
 * reference allocates in the Trainer / Mapper constructors
 * (Trainer.h:216-260, Mapper.h:138-178), including the cos/sin tables. */
int pink_b200_create(const pink_b200_config* cfg, pink_b200_ctx** out);
int pink_b200_destroy(pink_b200_ctx* ctx);

/* The neurons that live on this context's device: global neurons first + j * stride, j < count, with
 * stride = pink_b200_shard_stride(ctx).  count is N/world (+1 for the first N % world ranks), the sizes of
 * the reference's multi-GPU split (src/CudaLib/generate_euclidean_distance_matrix_first_step_multi_gpu.h:65-77).
 * By default the shards are interleaved (first = rank, stride = world_size), so that the neurons around any best
 * matching unit -- the ones an image rewrites -- are spread evenly over the ranks; option "sharding" = 1 selects
 * the reference's contiguous ranges (stride 1).  Mapping results are in this local order. */
int pink_b200_shard(const pink_b200_ctx* ctx, uint32_t* first, uint32_t* count);
uint32_t pink_b200_shard_stride(const pink_b200_ctx* ctx);
/* The reference's contiguous split as a pure host function (no context, no GPU). */
int pink_b200_shard_range(uint32_t n_neurons, uint32_t world_size, uint32_t rank, uint32_t* first, uint32_t* count);

/* Switches of a context, to be set after pink_b200_create and before pink_b200_comm_init /
 * pink_b200_set_som (no reference counterpart: the reference has one fixed launch sequence).  Unknown
 * names and values out of range return PINK_B200_EINVAL.
 *   "step_kernel"          0 (default) whole batches of training steps in one persistent kernel where the
 *                          geometry allows it; 1 two kernels per image (distance, update); 2 four kernels
 *                          per image (distance, best matching unit, work list, update)
 *   "sharding"             0 (default) interleaved neuron shards, 1 contiguous ranges as in the reference
 *   "exchange"             0 (default) per-rank records through peer memory where possible; 1 NCCL all-gather
 *   "rotation_sharing"     -1 (default) pairs of ranks share the rotation work; 0 every rank rotates every
 *                          image; g >= 2 groups of g consecutive ranks share
 *   "rotation_overlap"     1 puts the rotation kernels on a second, low-priority stream (default 0)
 *   "mma_pairs"            0 keeps the distance kernel from pairing blocks (default 1)
 *   "f32_filter"           0 computes float32 distances with the all-pairs exact kernel instead of the tensor-core
 *                          estimate + exact pass (default 1)
 *   "cooperative_launch"   0 launches the persistent kernel without the cooperative attribute (default 1).  Its
 *                          blocks wait for one another, so this is only for a device with nothing else running,
 *                          under a profiler that refuses cooperative launches; a block that is not resident
 *                          ends the batch with PINK_B200_ETIMEOUT instead of a hang
 *   "exchange_timeout_ms"  wall-clock limit of every device-side wait for another rank (default 20000).  The
 *                          ranks must enqueue each batch of steps within this time of one another. */
int pink_b200_set_option(pink_b200_ctx* ctx, const char* name, long long value);

/* ---- multi-GPU: one process per GPU, neuron shards, NCCL for the BMU exchange
 * (replaces the per-image cudaMemcpyPeer traffic of
 *  src/CudaLib/generate_euclidean_distance_matrix_first_step_multi_gpu.h:87-104,184-193). */

/* Rank 0 fills a 128-byte NCCL unique id; the caller distributes it. */
int pink_b200_comm_unique_id(void* id128);
/* Collective over all ranks of the job; required before training when world_size > 1. */
int pink_b200_comm_init(pink_b200_ctx* ctx, const void* id128);

/* ---- SOM and neighbourhood table ------------------------------------------- */

/* Upload the SOM (host, [N][P] float, the WHOLE map: each rank keeps its
 * shard) and build the distance operand.  Stands for the device copy taken at
 * construction, Trainer.h:219 / Mapper.h:140. */
int pink_b200_set_som(pink_b200_ctx* ctx, const float* host_som);
/* Write this rank's shard into its rows (first + j * stride) of host_som ([N][P]);
 * other rows are left untouched.  Stands for Trainer::update_som(), Trainer.h:306-309. */
int pink_b200_get_som(pink_b200_ctx* ctx, float* host_som);
/* Upload the N x N update-factor table F[bmu * N + n] the reference builds on
 * the host from the layout distance and the distribution function
 * (Trainer.h:69-76, uploaded at :243).  Each rank keeps its columns. */
int pink_b200_set_update_factors(pink_b200_ctx* ctx, const float* host_factors);

/* Host helpers (no GPU involved) for the tables the reference computes on the
 * host.  Number of neurons of a SOM grid: dim0 * dim1 (cartesian) or the
 * row-packed hexagon of side dim0 (HexagonalLayout.h:61-64). */
uint32_t pink_b200_som_size(uint32_t som_layout, uint32_t dim0, uint32_t dim1);
/* out[i * N + j] = layout.get_distance(i, j) (CartesianLayout.h:47-60,108-114;
 * HexagonalLayout.h:90-118). */
int pink_b200_som_distances(uint32_t som_layout, uint32_t dim0, uint32_t dim1, float* out);
/* out[i * N + j] = func(distance) if max_update_distance <= 0 or distance <
 * max_update_distance, else 0 -- the TrainerCommon loop (Trainer.h:69-76) for
 * the built-in functors (DistributionFunctor.cpp:18-59).  Callers with their
 * own distribution function fill the table themselves. */
int pink_b200_update_factors(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t func, float p0, float p1,
                             float max_update_distance, float* out);

/* The same without an N x N table (no reference counterpart; the reference evaluates its distribution function N^2
 * times and keeps N^2 floats, Trainer.h:69-76 -- 7.8 million calls and 31 MB for 2,791 neurons).  The map distance of
 * two neurons takes few distinct values: it depends only on the absolute coordinate differences (cartesian grids of
 * up to three dimensions; dim2 = 1 for two) or is the hop count (hexagonal; dim2 = 1).  pink_b200_distance_classes
 * returns their number and (if `distances` is not NULL) the distance of every class; a caller with its own
 * distribution function evaluates it once per class, applies the max_update_distance cut-off and hands the result to
 * pink_b200_set_update_lut.  pink_b200_update_lut does that for the built-in functors, pink_b200_set_update_function
 * both steps.  The factors are identical to the table's, bit for bit.  pink_b200_som_coordinates: the grid
 * position (x, y, z, 0 -- hexagonal: axial q, r) of every neuron as int16[N][4]. */
uint32_t pink_b200_distance_classes(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2, float* distances,
                                    uint32_t capacity);
int pink_b200_som_coordinates(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2, int16_t* out);
int pink_b200_update_lut(uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t func, float p0, float p1,
                         float max_update_distance, float* lut, uint32_t capacity);
int pink_b200_set_update_lut(pink_b200_ctx* ctx, uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                             const float* host_lut, uint32_t n_classes);
int pink_b200_set_update_function(pink_b200_ctx* ctx, uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                  uint32_t func, float p0, float p1, float max_update_distance);

/* The same two tables for a three-dimensional cartesian SOM of dim0 x dim1 x dim2
 * neurons (CartesianLayout<3>, CartesianLayout.h:116-123 for the position of an
 * array index; the command line tool's --som-depth > 1, main_gpu.cu:24-25). */
int pink_b200_som_distances_3d(uint32_t dim0, uint32_t dim1, uint32_t dim2, float* out);
int pink_b200_update_factors_3d(uint32_t dim0, uint32_t dim1, uint32_t dim2, uint32_t func, float p0, float p1,
                                float max_update_distance, float* out);

/* ---- training --------------------------------------------------------------
 * n sequential training steps; image i+1 sees the SOM updated by image i.
 * Stands for n calls of Trainer<...,true>::operator() (Trainer.h:263-304).
 * Asynchronous with respect to the host except for staging of host images;
 * results are observed through get_som / get_update_counts / synchronize. */
int pink_b200_train(pink_b200_ctx* ctx, const float* host_images, uint64_t n);
int pink_b200_train_device(pink_b200_ctx* ctx, const float* dev_images, uint64_t n);
/* Per-neuron BMU hit counters, [N] (all ranks hold the same totals only for
 * their own shard; other entries are zero).  Stands for get_update_info(),
 * Trainer.h:79, counted at :302-303. */
int pink_b200_get_update_counts(pink_b200_ctx* ctx, uint32_t* host_counts);
/* Optional: global BMU index of each of the last train call's images (host, [n]);
 * only the rank owning the BMU writes an entry, others read 0xFFFFFFFF. */
int pink_b200_get_bmu_log(pink_b200_ctx* ctx, uint32_t* host_bmus, uint64_t n);

/* ---- mapping ---------------------------------------------------------------
 * For each of n images: dist[i][j] = sqrt(min over transforms of the scaled
 * squared distance to local neuron j), rot[i][j] = the first transform
 * attaining it; j runs over this rank's shard (count entries per image).
 * Stands for n calls of Mapper<...,true>::operator() (Mapper.h:181-208). */
int pink_b200_map(pink_b200_ctx* ctx, const float* host_images, uint64_t n, float* host_dist, uint32_t* host_rot);
int pink_b200_map_device(pink_b200_ctx* ctx, const float* dev_images, uint64_t n, float* dev_dist, uint32_t* dev_rot);

/* Wait for all queued work of the context; surfaces asynchronous errors and
 * device-side time-outs. */
int pink_b200_synchronize(pink_b200_ctx* ctx);

/* The CUDA stream (cudaStream_t) the context launches on, for callers that
 * time or order work against it. */
void* pink_b200_stream(pink_b200_ctx* ctx);

/* Number of CUDA kernels the context has launched since it was created (the
 * reference has no counterpart; benchmarks report it). */
uint64_t pink_b200_launch_count(pink_b200_ctx* ctx);

/* How the ranks exchange their best-matching-unit records every step (no
 * reference counterpart: the reference trains on one GPU).  PEER: each rank
 * stores its record into every rank's memory over NVLink and the update kernel
 * waits for them (ranks on one node, one GPU each); PEER_SHARED_ROTATION: the
 * same, and the ranks also share the rotation work -- each computes the rotation
 * sets of its part of every batch of images and copies them into all ranks'
 * buffers; NCCL: an all-gather per step; NONE: a single rank or no communicator yet. */
enum { PINK_B200_EXCHANGE_NONE = 0, PINK_B200_EXCHANGE_NCCL = 1, PINK_B200_EXCHANGE_PEER = 2,
       PINK_B200_EXCHANGE_PEER_SHARED_ROTATION = 3 };
int pink_b200_exchange_kind(pink_b200_ctx* ctx);

/* Totals over all training steps of this context (this rank's shard): out[0] =
 * neurons that had a non-zero update factor, out[1] = neurons written back.
 * The reference rewrites every neuron (update_neurons.h:34-49); here a neuron
 * whose new values all equal the old ones bit for bit is read but not written. */
int pink_b200_get_update_stats(pink_b200_ctx* ctx, uint64_t* out);

/* Opt-in phase timing (the reference only has a wall clock around the whole
 * run, src/Pink/main.cpp:37-62).  After profile_begin, CUDA events on the
 * context's streams bracket the kernels of each of the next max_steps
 * training steps; profile_end waits for them and returns the summed device
 * time in milliseconds of {rotation sets (batched, overlapped with the steps),
 * distance, BMU + exchange, update} and the number of steps covered.  Event records perturb the pipeline slightly:
 * use it to apportion time between kernels, not to measure throughput. */
int pink_b200_profile_begin(pink_b200_ctx* ctx, uint32_t max_steps);
int pink_b200_profile_end(pink_b200_ctx* ctx, double ms_sum[4], uint64_t* steps);
/* After profile_end, for a context that trains with the persistent kernel (all zeros otherwise):
 * out[0] = mean device time of one launch in microseconds (CUDA events), out[1] = mean images per launch,
 * out[2..6] = mean microseconds per image, read from device-timer stamps of block 0, of: its own distance
 * tiles (TMA + MMA + epilogue), waiting for the other blocks at the first grid barrier, best matching unit
 * (+ exchange between ranks) and work list, rewriting its own neurons, waiting at the second grid barrier;
 * out[7] unused. */
int pink_b200_profile_detail(pink_b200_ctx* ctx, double out[8]);
/* The raw stamps behind it, [steps][blocks][12] words: nanoseconds of the device timer when (0) the image began,
 * (1) the block had reduced its own distance tiles, (2) it had passed the first grid barrier, (3) its work
 * list was built, (4) its own neurons were rewritten and stored, (5) it had passed the second grid barrier;
 * (6) neuron planes it rewrote, (7) distance tiles it computed; inside the phases: (8) first operand slice
 * arrived, (9) last MMA issued, (10) accumulators complete, (11) first neuron plane arrived.  *blocks and
 * *steps are always set; `out` may be NULL to ask for the sizes only. */
int pink_b200_profile_stamps(pink_b200_ctx* ctx, uint64_t* out, uint64_t capacity, uint32_t* blocks, uint64_t* steps);

/* float32 distances (mapping and training) run as an estimate of all N x T distances on the tensor cores followed
 * by exact sums for the transforms the estimate cannot rule out (option "f32_filter" = 0 computes all of them exactly instead; the
 * results are the same up to the summation order of the exact sums).  out[0] = pairs estimated so far,
 * out[1] = exact sums formed, out[2] = largest |estimate - exact| / (|a|^2 + |b|^2) seen among those,
 * out[3] = the error bound the selection assumes for that ratio. */
int pink_b200_map_filter_stats(pink_b200_ctx* ctx, double out[4]);

/* Ceiling of the integer tensor pipe as the distance kernels drive it: tera-operations per second of
 * tcgen05.mma kind::i8 (128 rows x n columns per CTA; pair != 0: CTA pairs, 256 x n per instruction) issued
 * back to back on operands already in shared memory, one CTA (pair) per SM.  n: multiple of 16, 16..256.
 * A measuring aid: the distance kernels' rates are quoted against it. */
int pink_b200_mma_i8_peak(int device, uint32_t n, int pair, double* tops);

/* ---- one process, several GPUs ------------------------------------------------
 * The reference's Trainer / Mapper use every visible GPU of the process on their own
 * (src/CudaLib/CudaLib.cu:56-76; neurons split over the GPUs with a host thread per extra GPU,
 * src/CudaLib/generate_euclidean_distance_matrix_first_step_multi_gpu.h:47-196).  A group is that for this
 * library: it owns one context per device and drives them from host threads of its own.
 *   training: the neurons are sharded over the devices (rank r on devices[r]) and the shards' records are
 *             exchanged through peer memory, as between processes;
 *   mapping:  every device holds the whole map and the images of a call are dealt to the devices in contiguous
 *             ranges; results are in the order of the images.  No communication.
 * `devices` lists CUDA ordinals; NULL takes the visible sm_100 devices (at most n_devices of them when n_devices
 * is not 0).  cfg->device, rank and world_size are ignored.  SOM, factors, counters and results are those of
 * the WHOLE map: a caller never sees the shards. */
typedef struct pink_b200_group pink_b200_group;
int pink_b200_device_count(void);                  /* visible sm_100 devices */
int pink_b200_group_create(const pink_b200_config* cfg, const int32_t* devices, uint32_t n_devices, pink_b200_group** out);
int pink_b200_group_destroy(pink_b200_group* group);
uint32_t pink_b200_group_size(const pink_b200_group* group);
int pink_b200_group_set_option(pink_b200_group* group, const char* name, long long value);
int pink_b200_group_set_som(pink_b200_group* group, const float* host_som);
int pink_b200_group_get_som(pink_b200_group* group, float* host_som);
int pink_b200_group_set_update_factors(pink_b200_group* group, const float* host_factors);
int pink_b200_group_set_update_lut(pink_b200_group* group, uint32_t som_layout, uint32_t dim0, uint32_t dim1, uint32_t dim2,
                                   const float* host_lut, uint32_t n_classes);
int pink_b200_group_train(pink_b200_group* group, const float* host_images, uint64_t n);
int pink_b200_group_get_update_counts(pink_b200_group* group, uint32_t* host_counts);
int pink_b200_group_synchronize(pink_b200_group* group);
int pink_b200_group_map(pink_b200_group* group, const float* host_images, uint64_t n, float* host_dist, uint32_t* host_rot);

/* Page-locked host memory for image and result buffers (the copies of pink_b200_train / pink_b200_map then run
 * asynchronously at full speed; pageable memory works too, slower).  The reference reads every image into
 * pageable memory (src/SelfOrganizingMapLib/DataIterator.h). */
int pink_b200_host_alloc(void** out, uint64_t bytes);
int pink_b200_host_free(void* ptr);

/* ---- single stages on device buffers (what the context calls internally) ---
 * Exposed for kernel-level parity tests and benchmarks.  `stream` is a
 * cudaStream_t (NULL = default stream).  Operand layout: integer modes use
 * rows of `row_stride` bytes (a multiple of 128, zero beyond K) per plane,
 * uint16 as two planes (high bytes, low bytes); float mode uses rows of
 * `row_stride` floats (a multiple of 32, zero beyond K). */

/* Row stride (in elements) the library uses for a distance length of K elements. */
uint32_t pink_b200_operand_stride(uint32_t K, uint32_t dist_type);

/* Rotation set of n_img images: base rotations (float, [n_img][max(R/4,1)][C][nd][nd],
 * may be NULL when shared memory holds a base) and the distance operand rows of
 * all T transforms with their sums of squares.  Stands for
 * SpatialTransformerGPU (src/CudaLib/generate_rotated_images.h:56-294) plus the
 * transform half of generate_euclidean_distance_matrix's crop/convert
 * (src/CudaLib/generate_euclidean_distance_matrix.h:86-112). */
int pink_b200_op_rotate(const pink_b200_config* cfg, const float* dev_images, uint32_t n_img,
                        float* dev_base, void* dev_b0, void* dev_b1, void* dev_bnorm, void* stream);

/* Same computation and arguments as pink_b200_op_rotate, for callers that cannot
 * allocate device memory: it calls neither cudaMalloc nor cudaFree nor any other
 * allocating routine.  (This entry has no counterpart in the reference.)
 * Who needs it: code that runs while the CUDA allocator must not be entered --
 * inside the callbacks of a caching allocator or memory pool, in a process that
 * has handed all device memory to its own arena, or in a loop that cannot afford
 * the implicit device synchronisation of cudaMalloc / cudaFree.
 * The table of rotation angles (the scratch pink_b200_op_rotate allocates per
 * call) lives in a fixed 32 KB device array inside the library, held by every GPU
 * that loads it until the process exits.  Limits and rules:
 *   - at most 16384 rotations (4096 per quadrant); more returns PINK_B200_EINVAL;
 *   - the first call on a device (and for each distance type) looks up the array's device address and
 *     loads the kernel; that first call may allocate inside the CUDA driver (module loading), so make one
 *     warm-up call per device and distance type before entering a region where allocation is forbidden;
 *     only later calls are allocation-free;
 *   - all calls share the one array (each overwrites the part it uses), so two
 *     calls whose GPU work may overlap -- different streams or host threads --
 *     race; serialise them.  The call returns after its work on `stream` is done. */
int pink_b200_op_rotate_static(const pink_b200_config* cfg, const float* dev_images, uint32_t n_img,
                               float* dev_base, void* dev_b0, void* dev_b1, void* dev_bnorm, void* stream);

/* SOM half of the crop/convert (generate_euclidean_distance_matrix.h:64-84). */
int pink_b200_op_quantize_som(const pink_b200_config* cfg, const float* dev_som, uint32_t n_neurons,
                              void* dev_a0, void* dev_a1, void* dev_anorm, void* stream);

/* Distance of every (neuron, transform) pair reduced to the per-neuron minimum
 * key (code << shift | transform; shift 32, or 16 for uint16), merged into
 * dev_keys with an unsigned minimum (fill with 0xFF bytes first).  dev_matrix
 * (nullable) receives the full [n_img][n][T] matrix: uint32 (uint8 mode),
 * uint64 (uint16), float (float).  Stands for
 * generate_euclidean_distance_matrix_first_step + _second_step
 * (src/CudaLib/generate_euclidean_distance_matrix_first_step.h:17-52,
 *  ..._second_step.h:43-62). */
int pink_b200_op_distance(uint32_t dist_type, uint32_t n_neurons, uint32_t n_transforms, uint32_t K,
                          const void* dev_a0, const void* dev_a1, const void* dev_anorm,
                          const void* dev_b0, const void* dev_b1, const void* dev_bnorm, uint32_t n_img,
                          unsigned long long* dev_keys, void* dev_matrix, void* stream);

/* Waits for the device and reports (then clears) a time-out recorded by a
 * pink_b200_op_distance launch: PINK_B200_OK or PINK_B200_ETIMEOUT. */
int pink_b200_op_status(void);

#ifdef __cplusplus
}
#endif
#endif /* PINK_B200_H */
