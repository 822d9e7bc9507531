// C ABI of the quantized-Linear operator: validation, dispatch, tensor-map encoding, grouped
// plans. Mirrors the host logic of Ops::linear / Ops::linear_activation
// (src/cuda/ops_blas.cpp:244-397 of the reference), int8_convrot_linear
// (src/cuda/int8_convrot.cu:579-751) and native_fp8_linear (ops_blas.cpp:153-225); where the
// reference throws CudaError this layer returns a status code and records a message.

#include "../../include/sdxlq.h"

#include "internal.cuh"
#include "quantize.cuh"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <string>
#include <tuple>
#include <vector>

namespace sdxlq {
cudaError_t launch_umma_gemm(const GemmLaunchParams& params, uint32_t grid, size_t dynamic_smem,
                             cudaStream_t stream, int device, bool pair, bool early_launch, int operand_class);
size_t umma_gemm_control_bytes();
cudaError_t launch_small_linear(const void* a, const void* b, const EpilogueParams& ep, uint32_t k_major,
                                cudaStream_t stream);
cudaError_t launch_bounded_wait_probe(uint32_t* error_word, long long limit_cycles, cudaStream_t stream);
cudaError_t launch_int8_plain_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t max_vectors,
                                   cudaStream_t stream, bool early_launch);
cudaError_t launch_int8_rotated256_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                        cudaStream_t stream, bool early_launch);
cudaError_t launch_int8_rotated_rows(const QuantInt8Launch& launch, uint32_t blocks, uint32_t threads,
                                     uint32_t stages, cudaStream_t stream, bool early_launch);
}  // namespace sdxlq

using namespace sdxlq;

namespace {

constexpr size_t kDefaultWorkspace = size_t(256) << 20;
constexpr uint32_t kMaxFp8Jobs = 4096;
constexpr size_t kNormPartialFloats = 256u * 1024u;     // scratch of sdxlq_group_norm_nhwc: partial sums (1 MiB; also the
                                                        // row statistics between the two LayerNorm -> FP8 launches) ...
constexpr size_t kNormMaxBatch = 1024;                  // ... then [batch, 64, 2] final statistics and [batch] counters
constexpr size_t kNormScratchBytes = kNormPartialFloats * sizeof(float) + kNormMaxBatch * 64 * 2 * sizeof(float) +
                                     kNormMaxBatch * sizeof(uint32_t);
constexpr size_t kSmemLimit = 232448;      // 227 KiB opt-in shared memory per CTA on sm_100

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

size_t align_up(size_t value, size_t alignment) { return (value + alignment - 1) / alignment * alignment; }

}  // namespace

struct sdxlq_context {
    int device = 0;
    cudaStream_t stream = nullptr;
    uint8_t* workspace = nullptr;
    size_t workspace_bytes = 0;
    float* norm_partials = nullptr;           // kNormPartialFloats floats: partial sums of sdxlq_group_norm_nhwc
    uint32_t* control = nullptr;           // [0] error word; from word 64: kMaxFp8Jobs amax words, then kMaxFp8Jobs
                                           // reader counters of the FP8 quantiser (all zero between calls)
    int sm_count = 148;
    uint8_t* staging = nullptr;            // pinned host image of the tables of a one-shot grouped call
    size_t staging_bytes = 0;
    cudaEvent_t staging_event = nullptr;   // completion of the last upload from `staging`
    int geglu_tile_n = 0;                     // tuning: accumulator tile width of GEGLU projections in grouped launches
                                              // (0: cost model). 128 lets the MMA issuer run three tiles ahead of the
                                              // GEGLU epilogues but measured slower (operand traffic, per-tile costs).
    int pair_mode = 0;                        // 0 never use CTA pairs (default: they measured no faster), 1 whenever
                                              // possible, -1 for traffic-bound launches only
    uint32_t diagnostic_skip = 0;             // SDXLQ_DIAGNOSTIC_SKIP: tuning aid, see GemmLaunchParams
    long long wait_limit_cycles = 4000000000LL;
    int forced_tile_n = 0;
    EncodeTiledFn encode = nullptr;
    uint32_t grouped_quant_threads = 0;       // tuning: block size of the rotated / general INT8 quantisers in grouped
                                              // launches (0: chosen per launch, see choose_quantiser_block)
    bool early_launch = true;                 // GEMM grids start while the quantiser before them drains (programmatic
                                              // dependent launch); the kernel waits before reading what it wrote
    sdxlq_int8_stats stats{};
    std::string last_error = "";
    // Optional per-kernel timing: CUDA event pairs recorded around each launch on the stream.
    bool profiling = false;
    struct TimedLaunch { int kernel_class; cudaEvent_t start; cudaEvent_t stop; int launches; };
    std::vector<TimedLaunch> timed;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> event_pool;
};

namespace {

// Records an event pair around the launches issued while it is alive (profiling mode only).
class LaunchTimer {
public:
    LaunchTimer(sdxlq_context* ctx, int kernel_class, int launches = 1) : ctx_(ctx) {
        if (!ctx_->profiling) return;
        std::pair<cudaEvent_t, cudaEvent_t> events{nullptr, nullptr};
        if (!ctx_->event_pool.empty()) {
            events = ctx_->event_pool.back();
            ctx_->event_pool.pop_back();
        } else if (cudaEventCreate(&events.first) != cudaSuccess || cudaEventCreate(&events.second) != cudaSuccess) {
            return;
        }
        entry_ = {kernel_class, events.first, events.second, launches};
        active_ = cudaEventRecord(entry_.start, ctx_->stream) == cudaSuccess;
    }
    ~LaunchTimer() {
        if (!active_) return;
        cudaEventRecord(entry_.stop, ctx_->stream);
        ctx_->timed.push_back(entry_);
    }
    LaunchTimer(const LaunchTimer&) = delete;
    LaunchTimer& operator=(const LaunchTimer&) = delete;

private:
    sdxlq_context* ctx_;
    sdxlq_context::TimedLaunch entry_{};
    bool active_ = false;
};

int fail(sdxlq_context* ctx, int status, const std::string& message) {
    if (ctx != nullptr) ctx->last_error = message;
    return status;
}

int fail_cuda(sdxlq_context* ctx, cudaError_t error, const char* where) {
    return fail(ctx, SDXLQ_ERR_CUDA, std::string(where) + ": " + cudaGetErrorString(error));
}

bool is_fp8(int32_t dtype) { return dtype == SDXLQ_FP8_E4M3 || dtype == SDXLQ_FP8_E5M2; }

bool valid_group(size_t group_size) {
    if (group_size < 4 || group_size > 256) return false;
    while (group_size > 1) {
        if (group_size % 4 != 0) return false;
        group_size /= 4;
    }
    return true;
}

uint32_t group_stages(uint32_t group_size) {
    uint32_t stages = 0;
    while (group_size > 1) { group_size /= 4; ++stages; }
    return stages;
}

// ---- validation: the checks of Ops::linear, int8_convrot_linear, fp8_weight_only_linear ----
int validate(sdxlq_context* ctx, const sdxlq_linear_desc& d) {
    const sdxlq_weight& w = d.weight;
    // An empty input (m == 0) is a no-op whose input and output buffers may be null.
    if (w.data == nullptr || (d.y == nullptr && d.m != 0)) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: null weight or output pointer");
    if (d.x == nullptr && d.xq == nullptr && d.m != 0) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: null input pointer");
    if (w.n == 0 || w.k == 0) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: empty weight");
    // Tile coordinates and the K-block count travel as 16-bit fields of a tile record.
    if (d.m > 0xFFFFull * kTileM || w.n > 0xFFFFull * 16 || w.k > 0xFFFFull * 64) {
        return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "linear dimensions exceed kernel integer range");
    }
    if (d.activation < SDXLQ_ACT_NONE || d.activation > SDXLQ_ACT_GEGLU) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: unknown activation");
    }
    if (d.activation != SDXLQ_ACT_NONE && d.bias == nullptr) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "fused linear bias activation requires a bias");
    }
    if (d.activation == SDXLQ_ACT_GEGLU && w.n % 2 != 0) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "fused linear bias GEGLU requires matching even-width FP16 tensors");
    }
    if (d.residual != nullptr && d.activation != SDXLQ_ACT_NONE) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: a residual is added to un-activated projections only");
    }
    if (w.dtype == SDXLQ_INT8) {
        if (w.scales == nullptr || w.scale_mode != SDXLQ_SCALE_PER_OUTPUT_CHANNEL) {
            return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 linear received incompatible tensors");
        }
        if (w.scale_count != w.n) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 linear feature or scale mismatch");
        if (w.convrot_group_size != 0 && (!valid_group(w.convrot_group_size) || w.k % w.convrot_group_size != 0)) {
            return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 linear has invalid ConvRot group metadata");
        }
        if (w.k % 4 != 0) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 Tensor Core linear requires K divisible by 4");
        if (w.layout != SDXLQ_ROW_MAJOR_NK) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "INT8 weights are row-major [N,K]");
        if (d.xq != nullptr && d.xq_scales == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: xq without xq_scales");
    } else if (is_fp8(w.dtype)) {
        if (w.scales == nullptr || (w.scale_count != 1 && w.scale_count != w.n)) {
            return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "FP8 weight has invalid scaling metadata");
        }
        if (w.scale_mode != SDXLQ_SCALE_TENSOR_WIDE && w.scale_mode != SDXLQ_SCALE_PER_OUTPUT_CHANNEL) {
            return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "FP8 weight has invalid scaling metadata");
        }
        if (w.layout != SDXLQ_ROW_MAJOR_NK && w.layout != SDXLQ_K_MAJOR_KN) {
            return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "FP8 weight has an unknown storage layout");
        }
        if (d.xq != nullptr && d.xq_scales == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: xq without xq_scales");
        if (d.acc_out != nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "acc_out is only defined for INT8 weights");
    } else if (w.dtype == SDXLQ_FP16) {
        if (w.layout != SDXLQ_ROW_MAJOR_NK) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "FP16 weights are row-major [N,K]");
        if (d.x == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "linear: null input pointer");
        if (d.acc_out != nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "acc_out is only defined for INT8 weights");
    } else {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "CUDA linear expects INT8, FP8 or FP16 weights");
    }
    return SDXLQ_OK;
}

// ---- tile shape ------------------------------------------------------------------------------
// Tile shape for one projection: accumulator width (columns) and whether a CTA pair
// (cta_group::2, 256-row tiles) works on it.
//  * A launch that fills the GPU several times over (grouped launches, big single projections) is
//    bound by operand traffic into shared memory. A single CTA moves (128 + t) bytes per k-byte for
//    128 * t MACs; a CTA pair moves (256 + t) for 256 * t. Cost of a projection per 128 rows:
//    ceil(N / t) * (128 + t), or ceil(N / t) * (128 + t / 2) for a pair (last-tile padding included).
//  * A launch of few tiles is bound by how many SMs get work: single CTAs, minimise waves * (t + 32).
struct TileChoice {
    uint32_t tile_n;
    bool pair;
};

TileChoice choose_tile(const sdxlq_context* ctx, uint32_t m, uint32_t n, bool geglu, bool grouped, uint32_t siblings = 1) {
    const uint32_t step = geglu ? 32 : 16;
    const uint32_t tiles_m = (m + kTileM - 1) / kTileM;
    const uint32_t sms = static_cast<uint32_t>(ctx->sm_count);
    const uint32_t columns = geglu ? n / 2 : n;            // GEGLU: a tile holds t/2 value + t/2 gate columns
    // `siblings`: problems of (about) this shape that share the launch (a small inline group)
    const uint64_t tiles_at_widest = static_cast<uint64_t>(siblings) * tiles_m * ((columns + (geglu ? 127 : 255)) / (geglu ? 128 : 256));
    const bool traffic_bound = grouped ? tiles_m >= 2 : tiles_at_widest >= 3ull * sms;
    // CTA pairs are opt-in (pair_mode): single calls, inline groups and plans all take them then.
    const bool pair_allowed = ctx->pair_mode != 0 && m > kTileM && (traffic_bound || ctx->pair_mode == 1);
    if (ctx->forced_tile_n >= 16) {
        const uint32_t forced = std::min<uint32_t>(kMaxTileN, static_cast<uint32_t>(ctx->forced_tile_n));
        const uint32_t pair_step = 32;
        if (pair_allowed) return TileChoice{std::max(pair_step, forced / pair_step * pair_step), true};
        return TileChoice{std::max(step, forced / step * step), false};
    }
    // Tuning override for the epilogue-heavy GEGLU tiles of a grouped launch (see geglu_tile_n).
    if (geglu && grouped && ctx->geglu_tile_n >= 32 && !pair_allowed) {
        return TileChoice{std::min<uint32_t>(kMaxTileN, static_cast<uint32_t>(ctx->geglu_tile_n) / 32u * 32u), false};
    }
    TileChoice best{step, false};
    double best_cost = 1e300;
    for (int pair = pair_allowed ? 1 : 0; pair >= 0; --pair) {
        const uint32_t tile_step = pair ? 32 : step;
        for (uint32_t tile_n = kMaxTileN; tile_n >= tile_step; tile_n -= tile_step) {
            const uint32_t per_tile = geglu ? tile_n / 2 : tile_n;
            const uint32_t tiles_n = (columns + per_tile - 1) / per_tile;
            double cost;
            if (traffic_bound || pair) {
                cost = static_cast<double>(tiles_n) * (128.0 + (pair ? tile_n / 2.0 : tile_n));
            } else {
                const uint64_t tiles = static_cast<uint64_t>(siblings) * tiles_m * tiles_n;
                const uint64_t waves = (tiles + sms - 1) / sms;
                cost = static_cast<double>(waves) * (tile_n + 32.0);
            }
            if (cost < best_cost) { best_cost = cost; best = TileChoice{tile_n, pair != 0}; }
            if (tile_n == tile_step) break;
        }
        if (pair) break;      // a pair is allowed only where it wins: traffic-bound launches
    }
    return best;
}

CUtensorMapDataType tensor_map_type(uint32_t kind) {
    return kind == KIND_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
}

bool encode_operand(const sdxlq_context* ctx, CUtensorMap* map, uint32_t kind, const void* pointer,
                    uint64_t rows, uint64_t k, uint32_t box_rows) {
    const uint64_t element = kind == KIND_F16 ? 2 : 1;
    const cuuint64_t dims[2] = {k, rows};
    const cuuint64_t strides[1] = {k * element};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTileKBytes / element), box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result = ctx->encode(map, tensor_map_type(kind), 2, const_cast<void*>(pointer), dims, strides,
                                        box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return result == CUDA_SUCCESS;
}

// ---- a prepared set of projections -------------------------------------------------------------
struct SmallCall {
    const void* a;
    const void* b;
    EpilogueParams ep;
    uint32_t k_major;
};

// INT8 quantiser jobs of one kernel flavour (one launch each).
struct Int8JobSet {
    std::vector<QuantInt8Job> jobs;
    uint32_t blocks = 0;
    uint32_t threads = 256;
    uint32_t max_vectors = 0;      // plain rows: most 16-byte vectors a lane holds
    uint32_t stage_mask = 0;       // rotated rows: bit s set when a job has `s` butterfly stages
};

enum Int8Flavour { INT8_GENERIC = 0, INT8_PLAIN = 1, INT8_ROTATED = 2, INT8_FLAVOURS = 3 };

struct Prepared {
    Int8JobSet int8[INT8_FLAVOURS];
    std::vector<QuantFp8Job> fp8_jobs;
    // GEMM problems by kernel flavour: [0] single CTA (128-row tiles), [1] CTA pair (256-row tiles)
    std::vector<GemmProblem> problems[2];
    std::vector<TileRef> tiles[2];
    uint32_t max_cta_b_rows[2] = {0, 0};     // most B rows one CTA stages (tile_n, or tile_n / 2 in a pair)
    std::vector<SmallCall> small;
    uint32_t fp8_blocks = 0;
    uint32_t int8_linears = 0;
    uint32_t int8_small = 0;
    size_t scratch_bytes = 0;
};

using QuantKey = std::tuple<const void*, uint64_t, uint64_t, uint32_t, uint32_t>;

// Block size of a single rotated / general quantiser launch: the best share of working threads, with the
// preference for 128-thread blocks that choose_quantiser_block gives grouped launches (measured 8 % faster at
// equal fill: X[16384, 1280] 20.2 us with 128 threads, 21.8 with 160, 22.9 with 256).
uint32_t best_int8_block(uint32_t threads_per_row) {
    uint32_t best = 256;
    double best_use = -1.0;
    for (uint32_t threads = 128; threads <= 256; threads += 32) {
        const uint32_t rows = threads / threads_per_row;
        if (rows == 0) continue;
        const double use = static_cast<double>(rows * threads_per_row) / threads * (threads == 128 ? 1.08 : 1.0);
        if (use > best_use + 1e-9) { best_use = use; best = threads; }
    }
    return best;
}

int add_int8_job(sdxlq_context* ctx, Prepared& prep, const void* x, bool x_is_f32, uint64_t m, uint64_t k,
                 uint32_t group, int8_t* xq, float* scales, bool grouped, const __half* gamma = nullptr,
                 const __half* beta = nullptr, float epsilon = 0.0f) {
    QuantInt8Job job{};
    job.gamma = gamma;           // a LayerNorm in front of the rotation: general kernel only
    job.beta = beta;
    job.epsilon = epsilon;
    job.x = x;
    job.xq = xq;
    job.scales = scales;
    job.m = static_cast<uint32_t>(m);
    job.k = static_cast<uint32_t>(k);
    job.stages = group_stages(group);
    job.threads_per_row = 4 * static_cast<uint32_t>((k + 255) / 256);
    if (job.threads_per_row > 256) return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "INT8 activation rows longer than 16384 are not supported");
    job.x_is_f32 = x_is_f32 ? 1 : 0;
    const size_t element = x_is_f32 ? 4 : 2;
    job.vector_ok = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && ((k * element) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(xq) % 8 == 0) && (k % 8 == 0) &&
                    reinterpret_cast<uintptr_t>(gamma) % 16 == 0 && reinterpret_cast<uintptr_t>(beta) % 16 == 0;
    // FP16 rows with a 16-byte pitch take the throughput kernels; everything else the general one.
    const bool fast = !x_is_f32 && job.vector_ok && gamma == nullptr;
    Int8Flavour flavour = INT8_GENERIC;
    if (fast && job.stages == 0 && k <= 5120) flavour = INT8_PLAIN;
    else if (fast && job.stages != 0) flavour = INT8_ROTATED;
    Int8JobSet& set = prep.int8[flavour];
    if (flavour == INT8_PLAIN) {
        job.rows_per_block = 8;                     // one warp per row, 256 threads
        set.max_vectors = std::max<uint32_t>(set.max_vectors, static_cast<uint32_t>((k / 8 + 31) / 32));
    } else {
        // grouped launches settle their block size once every job is known (choose_quantiser_block)
        const uint32_t threads = grouped ? 256 : best_int8_block(job.threads_per_row);
        set.threads = threads;
        job.rows_per_block = threads / job.threads_per_row;
        if (flavour == INT8_ROTATED) {
            // groups of 256 whose output rows are 16-byte aligned take the shared-memory exchange kernel
            job.pad = (job.stages == 4 && reinterpret_cast<uintptr_t>(xq) % 16 == 0 && k % 256 == 0) ? 1u : 0u;
            set.stage_mask |= job.pad != 0 ? (1u << 5) : (1u << job.stages);
        }
    }
    job.first_block = set.blocks;
    job.num_blocks = static_cast<uint32_t>((m + job.rows_per_block - 1) / job.rows_per_block);
    set.blocks += job.num_blocks;
    set.jobs.push_back(job);
    return SDXLQ_OK;
}

// Launches the INT8 activation quantisers of a prepared set: one launch per kernel flavour (and
// per rotation group size). `tables` holds the device copies of the job tables, or nulls.
int run_int8_quantisers(sdxlq_context* ctx, const Prepared& prep, QuantInt8Job* const tables[INT8_FLAVOURS],
                        uint16_t* const block_tables[INT8_FLAVOURS] = nullptr) {
    for (int flavour = 0; flavour < INT8_FLAVOURS; ++flavour) {
        const Int8JobSet& set = prep.int8[flavour];
        if (set.jobs.empty()) continue;
        cudaStream_t stream = ctx->stream;
        QuantInt8Launch launch{};
        launch.jobs = tables != nullptr ? tables[flavour] : nullptr;
        launch.block_jobs = launch.jobs != nullptr && block_tables != nullptr ? block_tables[flavour] : nullptr;
        launch.num_jobs = static_cast<uint32_t>(set.jobs.size());
        launch.single = set.jobs[0];
        if (launch.jobs == nullptr && set.jobs.size() != 1) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "internal: job table missing");
        cudaError_t error = cudaSuccess;
        const bool early = ctx->early_launch && !ctx->profiling;     // may be scheduled while the kernel before it drains
        LaunchTimer timer(ctx, SDXLQ_KERNEL_QUANT_INT8);
        if (flavour == INT8_GENERIC) {
            error = launch_rotate_quantize_int8(launch, set.blocks, set.threads, stream, early);
        } else if (flavour == INT8_PLAIN) {
            error = launch_int8_plain_rows(launch, set.blocks, set.max_vectors, stream, early);
        } else {
            for (uint32_t stages = 1; stages <= 4 && error == cudaSuccess; ++stages) {
                if (set.stage_mask & (1u << stages)) {
                    error = launch_int8_rotated_rows(launch, set.blocks, set.threads, stages, stream, early);
                }
            }
            if (error == cudaSuccess && (set.stage_mask & (1u << 5))) {
                error = launch_int8_rotated256_rows(launch, set.blocks, set.threads, stream, early);
            }
        }
        if (error != cudaSuccess) return fail_cuda(ctx, error, "INT8 activation quantise launch");
    }
    return SDXLQ_OK;
}

int int8_quantiser_launches(const Prepared& prep) {
    int launches = 0;
    for (int flavour = 0; flavour < INT8_FLAVOURS; ++flavour) {
        const Int8JobSet& set = prep.int8[flavour];
        if (set.jobs.empty()) continue;
        if (flavour != INT8_ROTATED) { ++launches; continue; }
        for (uint32_t stages = 1; stages <= 5; ++stages) launches += (set.stage_mask >> stages) & 1u;
    }
    return launches;
}

void add_fp8_job(Prepared& prep, const void* x, uint64_t count, uint32_t fmt, uint8_t* q, float* scale_out,
                 uint32_t* amax_in = nullptr) {
    QuantFp8Job job{};
    job.amax_in = amax_in;
    job.x = x;
    job.q = q;
    job.scale_out = scale_out;
    job.count = count;
    job.fmt = fmt;
    job.vector_ok = (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(q) % 8 == 0);
    job.first_block = prep.fp8_blocks;
    const uint64_t wanted = (count + 8191) / 8192;
    job.num_blocks = static_cast<uint32_t>(std::max<uint64_t>(1, std::min<uint64_t>(1184, wanted)));
    prep.fp8_blocks += job.num_blocks;
    prep.fp8_jobs.push_back(job);
}

void order_tiles(const sdxlq_context* ctx, const std::vector<GemmProblem>& problems, std::vector<TileRef>& tiles,
                 bool pair);

// One block size for all rotated (or general) quantiser jobs of a grouped launch. A row takes
// threads_per_row threads and a block holds whole rows, so the share of a block's threads that
// works depends on the block size (K = 5120: 80 threads per row fill 160 threads, 62 % of 128, 94 %
// of 256). Small blocks overlap one block's loads with another's arithmetic better: 128 threads
// measured 8 % faster than larger blocks at equal fill. Picks the size with the best fill weighted
// by the jobs' elements, then lays the jobs out in blocks of that size.
void choose_quantiser_block(const sdxlq_context* ctx, Int8JobSet& set) {
    if (set.jobs.empty()) return;
    uint32_t best_threads = 256;
    if (ctx->grouped_quant_threads != 0) {
        best_threads = ctx->grouped_quant_threads;
    } else {
        double best_score = -1.0;
        for (uint32_t threads = 128; threads <= 256; threads += 32) {
            double useful = 0.0, total = 0.0;
            for (const QuantInt8Job& job : set.jobs) {
                const uint32_t rows = threads / job.threads_per_row;
                const double elements = static_cast<double>(job.m) * job.k;
                useful += elements * (rows == 0 ? 0.0 : static_cast<double>(rows * job.threads_per_row) / threads);
                total += elements;
            }
            const double score = useful / total * (threads == 128 ? 1.08 : 1.0);
            if (score > best_score + 1e-9) { best_score = score; best_threads = threads; }
        }
    }
    // rows longer than the block cannot be split: fall back to the largest block
    for (const QuantInt8Job& job : set.jobs) if (job.threads_per_row > best_threads) best_threads = 256;
    set.threads = best_threads;
    set.blocks = 0;
    for (QuantInt8Job& job : set.jobs) {
        job.rows_per_block = best_threads / job.threads_per_row;
        job.first_block = set.blocks;
        job.num_blocks = (job.m + job.rows_per_block - 1) / job.rows_per_block;
        set.blocks += job.num_blocks;
    }
}

int prepare(sdxlq_context* ctx, const sdxlq_linear_desc* descs, size_t count, bool grouped, Prepared& prep) {
    std::map<QuantKey, std::pair<const void*, const float*>> shared_inputs;
    size_t scratch = 0;
    for (size_t index = 0; index < count; ++index) {
        const sdxlq_linear_desc& d = descs[index];
        const int status = validate(ctx, d);
        if (status != SDXLQ_OK) return status;
        if (d.m == 0) continue;
        const sdxlq_weight& w = d.weight;
        const uint32_t kind = w.dtype == SDXLQ_INT8 ? KIND_I8
                              : w.dtype == SDXLQ_FP8_E4M3 ? KIND_E4M3
                              : w.dtype == SDXLQ_FP8_E5M2 ? KIND_E5M2 : KIND_F16;
        const void* a = d.x;
        const float* a_scales = nullptr;
        if (kind == KIND_I8 || kind == KIND_E4M3 || kind == KIND_E5M2) {
            if (d.xq != nullptr) {
                a = d.xq;
                a_scales = d.xq_scales;
            } else {
                const uint32_t tag = kind == KIND_I8 ? w.convrot_group_size : 0;
                const QuantKey key{d.x, d.m, w.k, kind, tag};
                auto found = shared_inputs.find(key);
                if (found == shared_inputs.end()) {
                    const size_t q_offset = align_up(scratch, 256);
                    const size_t q_bytes = static_cast<size_t>(d.m) * w.k;
                    const size_t s_offset = align_up(q_offset + q_bytes, 256);
                    const size_t s_bytes = kind == KIND_I8 ? static_cast<size_t>(d.m) * sizeof(float) : sizeof(float);
                    scratch = s_offset + s_bytes;
                    if (scratch > ctx->workspace_bytes) {
                        return fail(ctx, SDXLQ_ERR_WORKSPACE, "workspace too small for the quantised activations");
                    }
                    uint8_t* q = ctx->workspace + q_offset;
                    float* s = reinterpret_cast<float*>(ctx->workspace + s_offset);
                    if (kind == KIND_I8) {
                        const int job_status = add_int8_job(ctx, prep, d.x, false, d.m, w.k, w.convrot_group_size,
                                                            reinterpret_cast<int8_t*>(q), s, grouped);
                        if (job_status != SDXLQ_OK) return job_status;
                    } else {
                        if (prep.fp8_jobs.size() >= kMaxFp8Jobs) {
                            return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "too many distinct FP8 inputs in one grouped call");
                        }
                        add_fp8_job(prep, d.x, static_cast<uint64_t>(d.m) * w.k, kind == KIND_E4M3 ? 0 : 1, q, s,
                                    static_cast<uint32_t*>(const_cast<void*>(d.x_amax)));
                    }
                    found = shared_inputs.emplace(key, std::make_pair(static_cast<const void*>(q), static_cast<const float*>(s))).first;
                }
                a = found->second.first;
                a_scales = found->second.second;
            }
        }

        EpilogueParams ep{};
        ep.y = static_cast<__half*>(d.y);
        ep.acc_out = d.acc_out;
        ep.a_scales = a_scales;
        ep.w_scales = w.scales;
        ep.bias = static_cast<const __half*>(d.bias);
        ep.residual = static_cast<const __half*>(d.residual);
        ep.y_amax = static_cast<uint32_t*>(d.y_amax);
        ep.m = static_cast<uint32_t>(d.m);
        ep.n = static_cast<uint32_t>(w.n);
        ep.k = static_cast<uint32_t>(w.k);
        const bool geglu = d.activation == SDXLQ_ACT_GEGLU;
        ep.n_out = geglu ? ep.n / 2 : ep.n;
        ep.kind = kind;
        ep.activation = static_cast<uint32_t>(d.activation);
        ep.w_scale_per_channel = (kind != KIND_F16 && w.scale_count != 1) ? 1 : 0;
        ep.vector_store_ok = (reinterpret_cast<uintptr_t>(d.y) % 16 == 0) && (ep.n_out % 8 == 0);
        ep.vector_meta_ok = (reinterpret_cast<uintptr_t>(w.scales) % 16 == 0) &&
                            (reinterpret_cast<uintptr_t>(d.bias) % 16 == 0) &&
                            (!geglu || ep.n_out % 8 == 0);

        const uint64_t element = kind == KIND_F16 ? 2 : 1;
        const bool tma_ok = w.layout == SDXLQ_ROW_MAJOR_NK && (w.k * element) % 16 == 0 &&
                            reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
                            reinterpret_cast<uintptr_t>(w.data) % 16 == 0;
        if (kind == KIND_I8) ++prep.int8_linears;
        if (!tma_ok) {
            if (kind == KIND_I8) ++prep.int8_small;
            prep.small.push_back(SmallCall{a, w.data, ep, w.layout == SDXLQ_K_MAJOR_KN ? 1u : 0u});
            continue;
        }

        GemmProblem problem{};
        problem.ep = ep;
        const TileChoice choice = choose_tile(ctx, ep.m, ep.n, geglu, grouped, grouped ? 1u : static_cast<uint32_t>(count));
        const int flavour = choice.pair ? 1 : 0;
        const uint32_t rows_per_tile = choice.pair ? 2 * kTileM : kTileM;
        problem.tile_n = choice.tile_n;
        const uint32_t per_tile = geglu ? problem.tile_n / 2 : problem.tile_n;
        problem.tiles_m = (ep.m + rows_per_tile - 1) / rows_per_tile;
        problem.tiles_n = (ep.n_out + per_tile - 1) / per_tile;
        problem.k_blocks = static_cast<uint32_t>((w.k * element + kTileKBytes - 1) / kTileKBytes);
        const uint32_t format = kind == KIND_I8 ? 1u : (kind == KIND_E5M2 ? 1u : 0u);
        // c_format: 2 = S32 for kind::i8, 1 = F32 otherwise; operands K-major; M = 128 (256 for a pair).
        problem.idesc = ((kind == KIND_I8 ? 2u : 1u) << 4) | (format << 7) | (format << 10) |
                        ((problem.tile_n >> 3) << 17) | ((rows_per_tile >> 4) << 24);
        // B box: the rows one TMA load brings in. A single CTA loads the whole tile (two boxes of
        // half the tile for GEGLU); each CTA of a pair loads half of the tile's rows.
        const uint32_t b_box_rows = choice.pair ? problem.tile_n / 2 : per_tile;
        if (!encode_operand(ctx, &problem.tmap_a, kind, a, ep.m, w.k, kTileM) ||
            !encode_operand(ctx, &problem.tmap_b, kind, w.data, w.n, w.k, b_box_rows)) {
            return fail(ctx, SDXLQ_ERR_CUDA, "cuTensorMapEncodeTiled rejected an operand");
        }
        prep.max_cta_b_rows[flavour] = std::max(prep.max_cta_b_rows[flavour], choice.pair ? problem.tile_n / 2 : problem.tile_n);
        const uint32_t problem_index = static_cast<uint32_t>(prep.problems[flavour].size());
        prep.problems[flavour].push_back(problem);
        if (grouped) {
            // n-major inside an m-tile keeps the CTAs of one wave on the same weight rows.
            for (uint32_t tn = 0; tn < problem.tiles_n; ++tn) {
                for (uint32_t tm = 0; tm < problem.tiles_m; ++tm) {
                    prep.tiles[flavour].push_back(make_tile_ref(problem, problem_index, tm, tn));
                }
            }
        }
    }
    for (int flavour = 0; flavour < 2; ++flavour) {
        if (!grouped || prep.problems[flavour].size() <= 1) continue;
        order_tiles(ctx, prep.problems[flavour], prep.tiles[flavour], flavour == 1);
    }
    if (grouped) {
        choose_quantiser_block(ctx, prep.int8[INT8_GENERIC]);
        choose_quantiser_block(ctx, prep.int8[INT8_ROTATED]);
    }
    prep.scratch_bytes = scratch;
    return SDXLQ_OK;
}

// Orders the tile list of a grouped launch. The persistent CTAs (or CTA pairs) walk it with a
// stride equal to their count, and a CTA overlaps the epilogue of tile i with the main loop of tile
// i + 1 (two accumulator buffers). Tiles whose epilogue outlasts their main loop (GEGLU with short
// K) are therefore alternated, one CTA-count block at a time, with tiles whose main loop dominates
// (long K); inside each class the longest tiles come first so that the walk ends evenly.
// Time model, fitted on B200: main loop ~ k_blocks * tile_n * 2.07e-3 us; epilogue ~ tile_n *
// 8.3e-3 us, or tile_n * 18e-3 us with the GEGLU epilogue. (Also tried: the cheapest epilogues in
// the last rounds so that less epilogue is exposed at the end of the launch; measured 2 % slower.)
void order_tiles(const sdxlq_context* ctx, const std::vector<GemmProblem>& problems, std::vector<TileRef>& tiles,
                 bool pair) {
    auto mainloop_time = [&](const TileRef& t) {
        const GemmProblem& p = problems[t.problem];
        return 2.07e-3 * p.k_blocks * p.tile_n;
    };
    auto epilogue_time = [&](const TileRef& t) {
        const GemmProblem& p = problems[t.problem];
        return (p.ep.activation == ACT_GEGLU ? 18.0e-3 : 8.3e-3) * p.tile_n;
    };
    std::vector<TileRef> epilogue_heavy, mainloop_heavy;
    for (const TileRef& t : tiles) (epilogue_time(t) > mainloop_time(t) ? epilogue_heavy : mainloop_heavy).push_back(t);
    auto longest_first = [&](const TileRef& l, const TileRef& r) {
        return std::max(mainloop_time(l), epilogue_time(l)) > std::max(mainloop_time(r), epilogue_time(r));
    };
    std::stable_sort(epilogue_heavy.begin(), epilogue_heavy.end(), longest_first);
    std::stable_sort(mainloop_heavy.begin(), mainloop_heavy.end(), longest_first);
    const size_t block = std::max<size_t>(1, pair ? ctx->sm_count / 2 : ctx->sm_count);
    const size_t total_e = epilogue_heavy.size(), total_m = mainloop_heavy.size();
    size_t taken_e = 0, taken_m = 0;
    tiles.clear();
    while (taken_e < total_e || taken_m < total_m) {
        // take the next block from the class that is behind its share of the list
        const bool take_e = taken_m >= total_m ||
                            (taken_e < total_e && taken_e * (total_e + total_m) <= (taken_e + taken_m) * total_e);
        std::vector<TileRef>& source = take_e ? epilogue_heavy : mainloop_heavy;
        size_t& taken = take_e ? taken_e : taken_m;
        const size_t count = std::min(block, source.size() - taken);
        tiles.insert(tiles.end(), source.begin() + taken, source.begin() + taken + count);
        taken += count;
    }
}

struct GemmGeometry {
    uint32_t stage_bytes;
    uint32_t num_stages;
    size_t dynamic_smem;
};

GemmGeometry gemm_geometry(uint32_t max_cta_b_rows) {
    GemmGeometry g{};
    g.stage_bytes = (kTileM + max_cta_b_rows) * kTileKBytes;
    const size_t control_bytes = umma_gemm_control_bytes();   // barriers, staged column operands, alignment slack
    g.num_stages = static_cast<uint32_t>(std::min<size_t>(8, (kSmemLimit - control_bytes) / g.stage_bytes));
    g.dynamic_smem = control_bytes + static_cast<size_t>(g.num_stages) * g.stage_bytes;
    return g;
}

// The launch header of the FP8 activation quantiser: one amax word and one reader counter per job,
// both zero when a call starts (the cast kernel puts them back, see fp8_cast_kernel).
QuantFp8Launch bind_fp8(sdxlq_context* ctx, const std::vector<QuantFp8Job>& jobs, const QuantFp8Job* device_jobs,
                        const uint16_t* block_jobs = nullptr) {
    QuantFp8Launch launch{};
    launch.block_jobs = device_jobs != nullptr ? block_jobs : nullptr;
    launch.amax_bits = ctx->control + 64;
    launch.done_counts = ctx->control + 64 + kMaxFp8Jobs;
    launch.jobs = device_jobs;
    launch.num_jobs = static_cast<uint32_t>(jobs.size());
    if (!jobs.empty()) launch.single = jobs[0];
    return launch;
}

// Launches the tensor-core GEMM of one kernel flavour: `problems` / `tiles` are the device tables
// of a grouped plan, or null when the (at most kInlineProblems) problems travel in the kernel
// parameters.
int run_gemm_flavour(sdxlq_context* ctx, const Prepared& prep, int flavour, const GemmProblem* problems,
                     const TileRef* tiles) {
    if (prep.problems[flavour].empty()) return SDXLQ_OK;
    const bool pair = flavour == 1;
    const GemmGeometry geometry = gemm_geometry(prep.max_cta_b_rows[flavour]);
    GemmLaunchParams params{};
    params.problems = problems;
    params.tiles = tiles;
    if (problems != nullptr) {
        params.num_tiles = static_cast<uint32_t>(prep.tiles[flavour].size());
    } else {
        const size_t count = prep.problems[flavour].size();
        if (count > kInlineProblems) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "internal: problem table missing");
        uint32_t tiles_so_far = 0;
        for (size_t i = 0; i < count; ++i) {
            params.inline_problems[i] = prep.problems[flavour][i];
            params.inline_tile_start[i] = tiles_so_far;
            tiles_so_far += params.inline_problems[i].tiles_m * params.inline_problems[i].tiles_n;
        }
        for (size_t i = count; i <= kInlineProblems; ++i) params.inline_tile_start[i] = tiles_so_far;
        params.inline_count = static_cast<uint32_t>(count);
        params.num_tiles = tiles_so_far;
    }
    params.num_stages = geometry.num_stages;
    params.stage_bytes = geometry.stage_bytes;
    params.b_offset = kTileM * kTileKBytes;
    params.error_word = ctx->control;
    params.wait_limit_cycles = ctx->wait_limit_cycles;
    params.diagnostic_skip = ctx->diagnostic_skip;
    const uint32_t sms = static_cast<uint32_t>(ctx->sm_count);
    const uint32_t grid = pair ? 2 * std::min<uint32_t>(params.num_tiles, sms / 2) : std::min<uint32_t>(params.num_tiles, sms);
    // the kernel instance compiled for one operand class when every problem of the launch has it
    int operand_class = -1;
    for (const GemmProblem& problem : prep.problems[flavour]) {
        const int this_class = problem.ep.kind == KIND_I8 ? 0 : (problem.ep.kind == KIND_F16 ? 2 : 1);
        if (operand_class == -1) operand_class = this_class;
        else if (operand_class != this_class) { operand_class = -2; break; }
    }
    LaunchTimer timer(ctx, SDXLQ_KERNEL_GEMM);
    const cudaError_t error = launch_umma_gemm(params, grid, geometry.dynamic_smem, ctx->stream, ctx->device, pair,
                                               ctx->early_launch && !ctx->profiling, operand_class);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "tensor-core GEMM launch");
    return SDXLQ_OK;
}

int run_small(sdxlq_context* ctx, const Prepared& prep) {
    for (const SmallCall& call : prep.small) {
        LaunchTimer timer(ctx, SDXLQ_KERNEL_SMALL);
        const cudaError_t status = launch_small_linear(call.a, call.b, call.ep, call.k_major, ctx->stream);
        if (status != cudaSuccess) return fail_cuda(ctx, status, "small linear launch");
    }
    return SDXLQ_OK;
}

void count_stats(sdxlq_context* ctx, const Prepared& prep) {
    ctx->stats.linear_calls += prep.int8_linears;
    ctx->stats.tensor_core_calls += prep.int8_linears - prep.int8_small;
    ctx->stats.dp4a_fallback_calls += prep.int8_small;
}

}  // namespace

struct sdxlq_group_plan {
    Prepared prep;
    uint8_t* slab = nullptr;                 // one device allocation holding every table below
    GemmProblem* device_problems[2] = {nullptr, nullptr};
    TileRef* device_tiles[2] = {nullptr, nullptr};
    QuantInt8Job* device_int8_jobs[INT8_FLAVOURS] = {nullptr, nullptr, nullptr};
    QuantFp8Job* device_fp8_jobs = nullptr;
    // the job of every block of the grouped quantiser launches (a block would otherwise search the job table)
    uint16_t* device_int8_block_jobs[INT8_FLAVOURS] = {nullptr, nullptr, nullptr};
    uint16_t* device_fp8_block_jobs = nullptr;
    int device = 0;
    const sdxlq_context* owner = nullptr;    // the tables hold addresses inside this context's workspace
};

namespace {

// Device tables of a prepared set, laid out back to back in one slab (128-byte aligned sections;
// tensor maps need 64).
struct TableLayout {
    size_t problems[2], tiles[2], int8_jobs[INT8_FLAVOURS], fp8_jobs, int8_block_jobs[INT8_FLAVOURS], fp8_block_jobs, total;
};

// Block -> job tables exist for launches of 2 to 65536 jobs (16-bit entries).
template <typename Job>
bool wants_block_table(const std::vector<Job>& jobs) { return jobs.size() > 1 && jobs.size() <= 65536; }

template <typename Job>
void fill_block_table(const std::vector<Job>& jobs, uint16_t* table) {
    for (size_t j = 0; j < jobs.size(); ++j) {
        for (uint32_t b = 0; b < jobs[j].num_blocks; ++b) table[jobs[j].first_block + b] = static_cast<uint16_t>(j);
    }
}

TableLayout layout_tables(const Prepared& prep) {
    TableLayout layout{};
    size_t offset = 0;
    auto place = [&](size_t bytes) { const size_t at = offset; offset = align_up(offset + bytes, 128); return at; };
    for (int f = 0; f < 2; ++f) layout.problems[f] = place(prep.problems[f].size() * sizeof(GemmProblem));
    for (int f = 0; f < 2; ++f) layout.tiles[f] = place(prep.tiles[f].size() * sizeof(TileRef));
    for (int f = 0; f < INT8_FLAVOURS; ++f) layout.int8_jobs[f] = place(prep.int8[f].jobs.size() * sizeof(QuantInt8Job));
    layout.fp8_jobs = place(prep.fp8_jobs.size() * sizeof(QuantFp8Job));
    for (int f = 0; f < INT8_FLAVOURS; ++f) {
        layout.int8_block_jobs[f] = place(wants_block_table(prep.int8[f].jobs) ? prep.int8[f].blocks * sizeof(uint16_t) : 0);
    }
    layout.fp8_block_jobs = place(wants_block_table(prep.fp8_jobs) ? prep.fp8_blocks * sizeof(uint16_t) : 0);
    layout.total = std::max<size_t>(offset, 128);
    return layout;
}

void fill_tables(const Prepared& prep, const TableLayout& layout, uint8_t* image) {
    auto copy = [&](size_t at, const auto& host) {
        if (!host.empty()) std::memcpy(image + at, host.data(), host.size() * sizeof(host[0]));
    };
    for (int f = 0; f < 2; ++f) { copy(layout.problems[f], prep.problems[f]); copy(layout.tiles[f], prep.tiles[f]); }
    for (int f = 0; f < INT8_FLAVOURS; ++f) copy(layout.int8_jobs[f], prep.int8[f].jobs);
    copy(layout.fp8_jobs, prep.fp8_jobs);
    for (int f = 0; f < INT8_FLAVOURS; ++f) {
        if (wants_block_table(prep.int8[f].jobs)) fill_block_table(prep.int8[f].jobs, reinterpret_cast<uint16_t*>(image + layout.int8_block_jobs[f]));
    }
    if (wants_block_table(prep.fp8_jobs)) fill_block_table(prep.fp8_jobs, reinterpret_cast<uint16_t*>(image + layout.fp8_block_jobs));
}

void bind_tables(sdxlq_group_plan* plan, const TableLayout& layout, uint8_t* slab) {
    const Prepared& prep = plan->prep;
    plan->slab = slab;
    for (int f = 0; f < 2; ++f) {
        plan->device_problems[f] = prep.problems[f].empty() ? nullptr : reinterpret_cast<GemmProblem*>(slab + layout.problems[f]);
        plan->device_tiles[f] = prep.tiles[f].empty() ? nullptr : reinterpret_cast<TileRef*>(slab + layout.tiles[f]);
    }
    for (int f = 0; f < INT8_FLAVOURS; ++f) {
        plan->device_int8_jobs[f] = prep.int8[f].jobs.empty() ? nullptr : reinterpret_cast<QuantInt8Job*>(slab + layout.int8_jobs[f]);
    }
    plan->device_fp8_jobs = prep.fp8_jobs.empty() ? nullptr : reinterpret_cast<QuantFp8Job*>(slab + layout.fp8_jobs);
    for (int f = 0; f < INT8_FLAVOURS; ++f) {
        plan->device_int8_block_jobs[f] =
            wants_block_table(prep.int8[f].jobs) ? reinterpret_cast<uint16_t*>(slab + layout.int8_block_jobs[f]) : nullptr;
    }
    plan->device_fp8_block_jobs = wants_block_table(prep.fp8_jobs) ? reinterpret_cast<uint16_t*>(slab + layout.fp8_block_jobs) : nullptr;
}

// Quantisers, GEMM flavours and small-shape kernels of a prepared set, in stream order.
int run_prepared(sdxlq_context* ctx, const Prepared& prep, const sdxlq_group_plan* tables) {
    int status = run_int8_quantisers(ctx, prep, tables != nullptr ? tables->device_int8_jobs : nullptr,
                                     tables != nullptr ? tables->device_int8_block_jobs : nullptr);
    if (status != SDXLQ_OK) return status;
    if (!prep.fp8_jobs.empty()) {
        const QuantFp8Launch launch = bind_fp8(ctx, prep.fp8_jobs, tables != nullptr ? tables->device_fp8_jobs : nullptr,
                                               tables != nullptr ? tables->device_fp8_block_jobs : nullptr);
        bool every_job_has_its_maximum = true;
        for (const QuantFp8Job& job : prep.fp8_jobs) every_job_has_its_maximum = every_job_has_its_maximum && job.amax_in != nullptr;
        LaunchTimer timer(ctx, SDXLQ_KERNEL_QUANT_FP8, every_job_has_its_maximum ? 1 : 2);
        const cudaError_t error = launch_fp8_quantize(launch, prep.fp8_blocks, ctx->stream, ctx->early_launch && !ctx->profiling,
                                                      every_job_has_its_maximum);
        if (error != cudaSuccess) return fail_cuda(ctx, error, "FP8 activation quantise launch");
    }
    for (int flavour = 0; flavour < 2; ++flavour) {
        status = run_gemm_flavour(ctx, prep, flavour, tables != nullptr ? tables->device_problems[flavour] : nullptr,
                                  tables != nullptr ? tables->device_tiles[flavour] : nullptr);
        if (status != SDXLQ_OK) return status;
    }
    status = run_small(ctx, prep);
    if (status != SDXLQ_OK) return status;
    count_stats(ctx, prep);
    return SDXLQ_OK;
}

// True when every kernel of the prepared set can take its operands from the kernel parameters: at
// most kInlineProblems GEMM problems per kernel flavour and one quantiser job per quantiser kernel.
bool fits_inline(const Prepared& prep) {
    if (prep.problems[1].size() > kInlineProblems || prep.problems[0].size() > kInlineProblems) return false;
    for (int f = 0; f < INT8_FLAVOURS; ++f) if (prep.int8[f].jobs.size() > 1) return false;
    return prep.fp8_jobs.size() <= 1;
}

}  // namespace

extern "C" {

int sdxlq_context_create(int device, void* stream, size_t workspace_bytes, sdxlq_context** out) {
    if (out == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    cudaError_t status = cudaSetDevice(device);
    if (status != cudaSuccess) return SDXLQ_ERR_CUDA;
    cudaDeviceProp properties{};
    status = cudaGetDeviceProperties(&properties, device);
    if (status != cudaSuccess) return SDXLQ_ERR_CUDA;
    if (properties.major != 10) return SDXLQ_ERR_UNSUPPORTED_SHAPE;   // sm_100a kernels only
    sdxlq_context* ctx = new (std::nothrow) sdxlq_context();
    if (ctx == nullptr) return SDXLQ_ERR_CUDA;
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(stream);
    ctx->sm_count = properties.multiProcessorCount;
    ctx->workspace_bytes = workspace_bytes == 0 ? kDefaultWorkspace : workspace_bytes;
    void* entry = nullptr;
    cudaDriverEntryPointQueryResult query{};
    status = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query);
    if (status != cudaSuccess || entry == nullptr) { delete ctx; return SDXLQ_ERR_CUDA; }
    ctx->encode = reinterpret_cast<EncodeTiledFn>(entry);
    if (cudaMalloc(&ctx->workspace, ctx->workspace_bytes) != cudaSuccess) { delete ctx; return SDXLQ_ERR_WORKSPACE; }
    const size_t control_bytes = (64 + 2 * kMaxFp8Jobs) * sizeof(uint32_t);
    if (cudaMalloc(&ctx->control, control_bytes) != cudaSuccess ||
        cudaMemset(ctx->control, 0, control_bytes) != cudaSuccess) {
        cudaFree(ctx->workspace);
        cudaFree(ctx->control);
        delete ctx;
        return SDXLQ_ERR_CUDA;
    }
    if (cudaEventCreateWithFlags(&ctx->staging_event, cudaEventDisableTiming) != cudaSuccess ||
        cudaMalloc(&ctx->norm_partials, kNormScratchBytes) != cudaSuccess ||
        cudaMemset(ctx->norm_partials, 0, kNormScratchBytes) != cudaSuccess) {
        if (ctx->staging_event != nullptr) cudaEventDestroy(ctx->staging_event);
        cudaFree(ctx->workspace);
        cudaFree(ctx->control);
        delete ctx;
        return SDXLQ_ERR_CUDA;
    }
    if (const char* text = std::getenv("SDXLQ_WAIT_LIMIT_CYCLES")) {
        const long long parsed = std::atoll(text);
        if (parsed > 0) ctx->wait_limit_cycles = parsed;
    }
    if (const char* text = std::getenv("SDXLQ_TILE_N")) ctx->forced_tile_n = std::atoi(text);
    if (const char* text = std::getenv("SDXLQ_PAIR")) ctx->pair_mode = std::atoi(text);
    if (const char* text = std::getenv("SDXLQ_GEGLU_TILE_N")) ctx->geglu_tile_n = std::atoi(text);
#ifdef SDXLQ_DIAGNOSTICS
    if (const char* text = std::getenv("SDXLQ_DIAGNOSTIC_SKIP")) ctx->diagnostic_skip = static_cast<uint32_t>(std::atoi(text));
#endif
    if (const char* text = std::getenv("SDXLQ_EARLY_LAUNCH")) ctx->early_launch = std::atoi(text) != 0;
    if (const char* text = std::getenv("SDXLQ_QUANT_THREADS")) {
        const int threads = std::atoi(text);
        if (threads >= 64 && threads <= 256 && threads % 32 == 0) ctx->grouped_quant_threads = static_cast<uint32_t>(threads);
    }
    *out = ctx;
    return SDXLQ_OK;
}

void sdxlq_context_destroy(sdxlq_context* ctx) {
    if (ctx == nullptr) return;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (auto& entry : ctx->timed) { cudaEventDestroy(entry.start); cudaEventDestroy(entry.stop); }
    for (auto& events : ctx->event_pool) { cudaEventDestroy(events.first); cudaEventDestroy(events.second); }
    if (ctx->staging_event != nullptr) cudaEventDestroy(ctx->staging_event);
    cudaFreeHost(ctx->staging);
    cudaFree(ctx->workspace);
    cudaFree(ctx->control);
    cudaFree(ctx->norm_partials);
    delete ctx;
}

int sdxlq_context_set_stream(sdxlq_context* ctx, void* stream) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    ctx->stream = static_cast<cudaStream_t>(stream);
    return SDXLQ_OK;
}

int sdxlq_context_set_tile_n(sdxlq_context* ctx, int tile_n) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    ctx->forced_tile_n = tile_n;
    return SDXLQ_OK;
}

int sdxlq_context_set_pair_mode(sdxlq_context* ctx, int mode) {
    if (ctx == nullptr || mode < -1 || mode > 1) return SDXLQ_ERR_INVALID_ARGUMENT;
    ctx->pair_mode = mode;
    return SDXLQ_OK;
}

int sdxlq_context_check(sdxlq_context* ctx) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    cudaError_t status = cudaStreamSynchronize(ctx->stream);
    if (status != cudaSuccess) return fail_cuda(ctx, status, "stream synchronize");
    uint32_t word = 0;
    status = cudaMemcpy(&word, ctx->control, sizeof(word), cudaMemcpyDeviceToHost);
    if (status != cudaSuccess) return fail_cuda(ctx, status, "error word read");
    if (word != 0) {
        cudaMemset(ctx->control, 0, sizeof(uint32_t));
        char text[96];
        std::snprintf(text, sizeof(text), "a bounded device-side wait ran out (code 0x%x)", word);
        return fail(ctx, SDXLQ_ERR_TIMEOUT, text);
    }
    return SDXLQ_OK;
}

const char* sdxlq_last_error(const sdxlq_context* ctx) { return ctx == nullptr ? "" : ctx->last_error.c_str(); }

const char* sdxlq_status_string(int status) {
    switch (status) {
    case SDXLQ_OK: return "ok";
    case SDXLQ_ERR_INVALID_ARGUMENT: return "invalid argument";
    case SDXLQ_ERR_UNSUPPORTED_SHAPE: return "unsupported shape";
    case SDXLQ_ERR_TIMEOUT: return "device wait timed out";
    case SDXLQ_ERR_CUDA: return "CUDA error";
    case SDXLQ_ERR_WORKSPACE: return "workspace too small";
    default: return "unknown status";
    }
}

int sdxlq_get_stats(const sdxlq_context* ctx, sdxlq_int8_stats* out) {
    if (ctx == nullptr || out == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    *out = ctx->stats;
    return SDXLQ_OK;
}

int sdxlq_valid_convrot_group_size(size_t group_size) { return valid_group(group_size) ? 1 : 0; }

const char* sdxlq_build_info(void) {
#ifdef SDXLQ_DIAGNOSTICS
    return "sdxlq sm_100a tcgen05/TMA cta_group::1 128xN + cta_group::2 256xN (diagnostic switches built in)";
#else
    return "sdxlq sm_100a tcgen05/TMA cta_group::1 128xN + cta_group::2 256xN";
#endif
}

size_t sdxlq_workspace_bytes(const sdxlq_linear_desc* descs, size_t count) {
    if (descs == nullptr) return 0;
    std::map<QuantKey, int> seen;
    size_t scratch = 0;
    for (size_t index = 0; index < count; ++index) {
        const sdxlq_linear_desc& d = descs[index];
        const sdxlq_weight& w = d.weight;
        if (d.m == 0 || d.xq != nullptr || w.dtype == SDXLQ_FP16) continue;
        const uint32_t kind = w.dtype == SDXLQ_INT8 ? KIND_I8 : (w.dtype == SDXLQ_FP8_E4M3 ? KIND_E4M3 : KIND_E5M2);
        const QuantKey key{d.x, d.m, w.k, kind, kind == KIND_I8 ? w.convrot_group_size : 0u};
        if (!seen.emplace(key, 1).second) continue;
        const size_t q_offset = align_up(scratch, 256);
        const size_t s_offset = align_up(q_offset + static_cast<size_t>(d.m) * w.k, 256);
        scratch = s_offset + (kind == KIND_I8 ? static_cast<size_t>(d.m) * sizeof(float) : sizeof(float));
    }
    return scratch;
}

int sdxlq_linear(sdxlq_context* ctx, const sdxlq_linear_desc* desc) {
    if (ctx == nullptr || desc == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    Prepared prep;
    const int status = prepare(ctx, desc, 1, false, prep);
    if (status != SDXLQ_OK) return status;
    return run_prepared(ctx, prep, nullptr);
}

int sdxlq_group_plan_create(sdxlq_context* ctx, const sdxlq_linear_desc* descs, size_t count,
                            sdxlq_group_plan** out) {
    if (ctx == nullptr || out == nullptr || (descs == nullptr && count != 0)) return SDXLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    sdxlq_group_plan* plan = new (std::nothrow) sdxlq_group_plan();
    if (plan == nullptr) return SDXLQ_ERR_CUDA;
    plan->device = ctx->device;
    plan->owner = ctx;
    const int status = prepare(ctx, descs, count, true, plan->prep);
    if (status != SDXLQ_OK) { delete plan; return status; }
    const TableLayout layout = layout_tables(plan->prep);
    std::vector<uint8_t> image(layout.total, 0);
    fill_tables(plan->prep, layout, image.data());
    uint8_t* slab = nullptr;
    if (cudaMalloc(reinterpret_cast<void**>(&slab), layout.total) != cudaSuccess ||
        cudaMemcpy(slab, image.data(), layout.total, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaFree(slab);
        delete plan;
        return fail(ctx, SDXLQ_ERR_CUDA, "grouped plan: device table allocation failed");
    }
    bind_tables(plan, layout, slab);
    *out = plan;
    return SDXLQ_OK;
}

int sdxlq_group_plan_run(sdxlq_context* ctx, sdxlq_group_plan* plan) {
    if (ctx == nullptr || plan == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (plan->owner != ctx) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT,
                    "grouped plan belongs to another context (its tables address that context's workspace)");
    }
    return run_prepared(ctx, plan->prep, plan);
}

int sdxlq_group_plan_launches(const sdxlq_group_plan* plan) {
    if (plan == nullptr) return 0;
    const Prepared& prep = plan->prep;
    return int8_quantiser_launches(prep) + (prep.fp8_jobs.empty() ? 0 : 2) + (prep.problems[0].empty() ? 0 : 1) + (prep.problems[1].empty() ? 0 : 1) +
           static_cast<int>(prep.small.size());
}

void sdxlq_group_plan_destroy(sdxlq_group_plan* plan) {
    if (plan == nullptr) return;
    cudaSetDevice(plan->device);
    cudaFree(plan->slab);
    delete plan;
}

int sdxlq_linear_grouped(sdxlq_context* ctx, const sdxlq_linear_desc* descs, size_t count) {
    if (ctx == nullptr || (descs == nullptr && count != 0)) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (count == 0) return SDXLQ_OK;
    // Small groups (the three attention projections of one input): everything travels in the kernel
    // parameters; no table, no allocation, nothing that a stream capture could not record.
    if (count <= kInlineProblems) {
        Prepared prep;
        const int status = prepare(ctx, descs, count, false, prep);
        if (status != SDXLQ_OK) return status;
        if (fits_inline(prep)) return run_prepared(ctx, prep, nullptr);
    }
    // Larger groups: tables go to the device through the context's pinned staging buffer and a
    // stream-ordered allocation that is released, in stream order, behind the kernels that read it.
    // The call returns without waiting for the GPU; it only waits for the previous grouped call's
    // table upload before it overwrites the staging buffer.
    if (ctx->staging_event == nullptr) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "grouped calls need a context made by sdxlq_context_create");
    }
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->stream, &capture) != cudaSuccess || capture != cudaStreamCaptureStatusNone) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT,
                    "a grouped call with device tables cannot be captured: build a plan before the capture and run that");
    }
    sdxlq_group_plan plan;
    plan.device = ctx->device;
    plan.owner = ctx;
    int status = prepare(ctx, descs, count, true, plan.prep);
    if (status != SDXLQ_OK) return status;
    const TableLayout layout = layout_tables(plan.prep);
    cudaError_t error = cudaEventSynchronize(ctx->staging_event);
    if (error == cudaSuccess && layout.total > ctx->staging_bytes) {
        cudaFreeHost(ctx->staging);
        ctx->staging = nullptr;
        ctx->staging_bytes = 0;
        const size_t wanted = align_up(layout.total * 2, size_t(1) << 20);
        error = cudaMallocHost(reinterpret_cast<void**>(&ctx->staging), wanted);
        if (error == cudaSuccess) ctx->staging_bytes = wanted;
    }
    if (error != cudaSuccess) return fail_cuda(ctx, error, "grouped call: table staging");
    fill_tables(plan.prep, layout, ctx->staging);
    uint8_t* slab = nullptr;
    error = cudaMallocAsync(reinterpret_cast<void**>(&slab), layout.total, ctx->stream);
    if (error == cudaSuccess) error = cudaMemcpyAsync(slab, ctx->staging, layout.total, cudaMemcpyHostToDevice, ctx->stream);
    if (error == cudaSuccess) error = cudaEventRecord(ctx->staging_event, ctx->stream);
    if (error != cudaSuccess) {
        if (slab != nullptr) cudaFreeAsync(slab, ctx->stream);
        return fail_cuda(ctx, error, "grouped call: table upload");
    }
    bind_tables(&plan, layout, slab);
    status = run_prepared(ctx, plan.prep, &plan);
    error = cudaFreeAsync(slab, ctx->stream);        // takes effect after the kernels above, in stream order
    if (status == SDXLQ_OK && error != cudaSuccess) status = fail_cuda(ctx, error, "grouped call: table release");
    return status;
}

int sdxlq_quantize_act_int8(sdxlq_context* ctx, const void* x, int32_t x_dtype, uint64_t m, uint64_t k,
                            uint32_t convrot_group_size, int8_t* xq, float* scales) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (x == nullptr || xq == nullptr || scales == nullptr || k == 0) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "quantize_act_int8: null pointer or empty row");
    }
    if (x_dtype != SDXLQ_FP16 && x_dtype != SDXLQ_FP32) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 linear received incompatible tensors");
    }
    if (convrot_group_size != 0 && (!valid_group(convrot_group_size) || k % convrot_group_size != 0)) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 linear has invalid ConvRot group metadata");
    }
    if (m > 0x7FFFFFFFull || k > 0x7FFFFFFFull) return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "quantize_act_int8: dimensions too large");
    if (m == 0) return SDXLQ_OK;
    Prepared prep;
    const int status = add_int8_job(ctx, prep, x, x_dtype == SDXLQ_FP32, m, k, convrot_group_size, xq, scales, false);
    if (status != SDXLQ_OK) return status;
    return run_int8_quantisers(ctx, prep, nullptr);
}

int sdxlq_quantize_act_fp8(sdxlq_context* ctx, const void* x_f16, uint64_t count, int32_t fmt, uint8_t* q,
                           float* scale) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (x_f16 == nullptr || q == nullptr || scale == nullptr || !is_fp8(fmt)) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "FP8 activation quantization requires float16 input and an FP8 destination");
    }
    Prepared prep;
    add_fp8_job(prep, x_f16, count, fmt == SDXLQ_FP8_E4M3 ? 0 : 1, q, scale);
    const QuantFp8Launch launch = bind_fp8(ctx, prep.fp8_jobs, nullptr);
    LaunchTimer timer(ctx, SDXLQ_KERNEL_QUANT_FP8, 2);
    const cudaError_t error = launch_fp8_quantize(launch, prep.fp8_blocks, ctx->stream, ctx->early_launch && !ctx->profiling, false);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "FP8 activation quantise launch");
    return SDXLQ_OK;
}

int sdxlq_layer_norm(sdxlq_context* ctx, const sdxlq_layer_norm_desc* desc) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (desc == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "layer_norm: null descriptor");
    const sdxlq_layer_norm_desc& d = *desc;
    if (d.width == 0) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "layer_norm requires a non-empty last dimension");
    if (d.rows == 0) return SDXLQ_OK;
    if (d.x == nullptr || d.gamma == nullptr || d.beta == nullptr) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "layer_norm: null input, weight or bias");
    }
    if (d.rows > 0x7FFFFFFFull || d.width > 0x7FFFFFFFull) {
        return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "layer_norm: dimensions too large");
    }
    const auto aligned = [](const void* pointer, uintptr_t bytes) { return reinterpret_cast<uintptr_t>(pointer) % bytes == 0; };
    // what the warp-per-row kernels take: rows of 16-byte vectors that fit a warp's registers
    const bool row_kernel_ok = d.width % 8 == 0 && d.width <= 2048 && aligned(d.x, 16) && aligned(d.gamma, 16) && aligned(d.beta, 16);
    LayerNormLaunch launch{};
    launch.x = static_cast<const __half*>(d.x);
    launch.gamma = static_cast<const __half*>(d.gamma);
    launch.beta = static_cast<const __half*>(d.beta);
    launch.rows = static_cast<uint32_t>(d.rows);
    launch.width = static_cast<uint32_t>(d.width);
    launch.epsilon = d.epsilon;

    if (d.out_dtype == SDXLQ_INT8) {
        if (d.xq == nullptr || d.xq_scales == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "layer_norm: null quantised output");
        if (d.convrot_group_size != 0 && (!valid_group(d.convrot_group_size) || d.width % d.convrot_group_size != 0)) {
            return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 linear has invalid ConvRot group metadata");
        }
        if (row_kernel_ok && d.convrot_group_size == 0 && aligned(d.xq, 8)) {
            // one launch: normalise, per-row maximum, cast
            launch.q = static_cast<uint8_t*>(d.xq);
            launch.scale_out = d.xq_scales;
            LaunchTimer timer(ctx, SDXLQ_KERNEL_LAYER_NORM);
            const cudaError_t error = launch_layer_norm_int8(launch, ctx->stream, ctx->early_launch && !ctx->profiling);
            if (error != cudaSuccess) return fail_cuda(ctx, error, "layer_norm launch");
            return SDXLQ_OK;
        }
        const size_t scratch = static_cast<size_t>(d.rows) * d.width * sizeof(__half);
        const void* source = d.x;
        const __half* gamma = static_cast<const __half*>(d.gamma);
        const __half* beta = static_cast<const __half*>(d.beta);
        if (row_kernel_ok && scratch <= ctx->workspace_bytes) {
            // rotated rows: the normalised FP16 tensor goes through the workspace (it stays in L2 for
            // the sizes of this model) and the throughput rotation kernels read it from there
            launch.y = reinterpret_cast<__half*>(ctx->workspace);
            LaunchTimer timer(ctx, SDXLQ_KERNEL_LAYER_NORM);
            const cudaError_t error = launch_layer_norm_f16(launch, ctx->stream, ctx->early_launch && !ctx->profiling);
            if (error != cudaSuccess) return fail_cuda(ctx, error, "layer_norm launch");
            source = ctx->workspace;
            gamma = beta = nullptr;
        }
        // otherwise (odd widths, rows past 2048 elements, no room): the general quantiser normalises
        // the row itself before it rotates it
        Prepared prep;
        const int status = add_int8_job(ctx, prep, source, false, d.rows, d.width, d.convrot_group_size,
                                        static_cast<int8_t*>(d.xq), d.xq_scales, false, gamma, beta, d.epsilon);
        if (status != SDXLQ_OK) return status;
        return run_int8_quantisers(ctx, prep, nullptr);
    }
    const bool fp8 = is_fp8(d.out_dtype);
    if (!fp8 && d.out_dtype != SDXLQ_FP16) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "layer_norm: unknown output type");
    void* const destination = fp8 ? d.xq : d.y;
    if (destination == nullptr || (fp8 && d.xq_scales == nullptr)) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "layer_norm: null output");
    }
    if (!row_kernel_ok || !aligned(destination, fp8 ? 8 : 16)) {
        return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE,
                    "layer_norm: rows must be 16-byte aligned, a multiple of 8 and at most 2048 elements wide");
    }
    launch.y = static_cast<__half*>(d.y);
    launch.q = static_cast<uint8_t*>(d.xq);
    launch.scale_out = d.xq_scales;
    launch.amax_bits = ctx->control + 64;
    launch.done_count = ctx->control + 64 + kMaxFp8Jobs;
    launch.fmt = d.out_dtype == SDXLQ_FP8_E5M2 ? 1u : 0u;
    // the normalisation scratch doubles as the rows' (mean, inverse deviation) between the two FP8 launches
    if (fp8 && ctx->norm_partials != nullptr && d.rows * sizeof(float2) <= kNormPartialFloats * sizeof(float)) {
        launch.row_stats = reinterpret_cast<float2*>(ctx->norm_partials);
    }
    LaunchTimer timer(ctx, SDXLQ_KERNEL_LAYER_NORM, fp8 ? 2 : 1);
    const cudaError_t error = fp8 ? launch_layer_norm_fp8(launch, ctx->stream, ctx->early_launch && !ctx->profiling)
                                  : launch_layer_norm_f16(launch, ctx->stream, ctx->early_launch && !ctx->profiling);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "layer_norm launch");
    return SDXLQ_OK;
}

int sdxlq_group_norm_nhwc(sdxlq_context* ctx, const sdxlq_group_norm_desc* desc) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (desc == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "group_norm: null descriptor");
    const sdxlq_group_norm_desc& d = *desc;
    if (d.batch == 0 || d.rows == 0) return SDXLQ_OK;
    if (d.x == nullptr || d.y == nullptr || d.gamma == nullptr || d.beta == nullptr) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "group_norm: null input, output, weight or bias");
    }
    if (d.groups == 0 || d.channels == 0 || d.channels % d.groups != 0) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "CUDA group_norm channels must be divisible by groups");
    }
    const auto aligned = [](const void* pointer) { return pointer == nullptr || reinterpret_cast<uintptr_t>(pointer) % 16 == 0; };
    if (d.groups > 64 || d.channels % 8 != 0 || d.channels > group_norm_max_channels() || d.batch > kNormMaxBatch ||
        d.rows > 0x7FFFFFFFull || !aligned(d.x) || !aligned(d.y) || !aligned(d.gamma) || !aligned(d.beta) || !aligned(d.channel_bias)) {
        return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE,
                    "group_norm: a multiple of 8 channels (at most 3072) with 16-byte aligned rows, at most 64 groups and 1024 images");
    }
    if (ctx->norm_partials == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "group_norm needs a context made by sdxlq_context_create");
    // enough blocks to fill the GPU a few times over; the partial sums of a launch must fit the scratch
    const uint64_t capacity = kNormPartialFloats / (2ull * d.groups);            // (batch x chunks) pairs of sums
    uint64_t chunks = std::max<uint64_t>(1, static_cast<uint64_t>(ctx->sm_count) * 4 / d.batch);
    chunks = std::min<uint64_t>(chunks, std::max<uint64_t>(1, d.rows / 8));
    chunks = std::min<uint64_t>(chunks, std::max<uint64_t>(1, capacity / d.batch));
    if (d.batch > capacity) return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "group_norm: batch too large for the scratch");
    GroupNormLaunch launch{};
    launch.x = static_cast<const __half*>(d.x);
    launch.channel_bias = static_cast<const __half*>(d.channel_bias);
    launch.gamma = static_cast<const __half*>(d.gamma);
    launch.beta = static_cast<const __half*>(d.beta);
    launch.y = static_cast<__half*>(d.y);
    launch.partials = ctx->norm_partials;
    launch.finals = ctx->norm_partials + kNormPartialFloats;
    launch.counters = reinterpret_cast<uint32_t*>(ctx->norm_partials + kNormPartialFloats + kNormMaxBatch * 64 * 2);
    launch.batch = static_cast<uint32_t>(d.batch);
    launch.rows = static_cast<uint32_t>(d.rows);
    launch.channels = static_cast<uint32_t>(d.channels);
    launch.groups = d.groups;
    launch.rows_per_chunk = static_cast<uint32_t>((d.rows + chunks - 1) / chunks);
    chunks = (d.rows + launch.rows_per_chunk - 1) / launch.rows_per_chunk;
    launch.silu = d.silu != 0 ? 1u : 0u;
    launch.epsilon = d.epsilon;
    LaunchTimer timer(ctx, SDXLQ_KERNEL_HARNESS, 2);
    const cudaError_t error = launch_group_norm_nhwc(launch, static_cast<uint32_t>(chunks), ctx->stream);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "group_norm launch");
    return SDXLQ_OK;
}

int sdxlq_harness_bias_residual_add(sdxlq_context* ctx, const void* x, const void* bias, const void* residual, void* y,
                                    uint64_t rows, uint64_t channels) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (rows == 0 || channels == 0) return SDXLQ_OK;
    if (x == nullptr || bias == nullptr || residual == nullptr || y == nullptr) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "CUDA add requires matching FP16 tensors");
    }
    const auto aligned = [](const void* pointer) { return reinterpret_cast<uintptr_t>(pointer) % 16 == 0; };
    if (channels % 8 != 0 || channels > 0x7FFFFFFFull || !aligned(x) || !aligned(bias) || !aligned(residual) || !aligned(y)) {
        return fail(ctx, SDXLQ_ERR_UNSUPPORTED_SHAPE, "bias_residual_add: 16-byte aligned rows of a multiple of 8 channels");
    }
    LaunchTimer timer(ctx, SDXLQ_KERNEL_HARNESS);
    const cudaError_t error = launch_bias_residual_add(static_cast<const __half*>(x), static_cast<const __half*>(bias),
                                                       static_cast<const __half*>(residual), static_cast<__half*>(y), rows,
                                                       static_cast<uint32_t>(channels), static_cast<uint32_t>(ctx->sm_count), ctx->stream);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "bias_residual_add launch");
    return SDXLQ_OK;
}

int sdxlq_pack_weight_int8(sdxlq_context* ctx, const void* src, int32_t src_dtype, uint64_t n, uint64_t k,
                           uint32_t convrot_group_size, int8_t* dst, float* scales) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (src == nullptr || dst == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "pack_weight_int8: null pointer");
    if (n == 0 || k == 0) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 weight cannot be empty");
    if (src_dtype == SDXLQ_INT8) {
        const cudaError_t error = cudaMemcpyAsync(dst, src, n * k, cudaMemcpyDeviceToDevice, ctx->stream);
        if (error != cudaSuccess) return fail_cuda(ctx, error, "prequantised INT8 weight copy");
        return SDXLQ_OK;
    }
    if (src_dtype != SDXLQ_FP16 && src_dtype != SDXLQ_FP32) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "native INT8 loading requires I8, F16 or F32 weights");
    }
    if (convrot_group_size != 0 && !valid_group(convrot_group_size)) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "INT8 ConvRot group size must be a power of four between 4 and 256");
    }
    if (convrot_group_size != 0 && k % convrot_group_size != 0) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "ConvRot group size does not divide the weight's input features");
    }
    return sdxlq_quantize_act_int8(ctx, src, src_dtype, n, k, convrot_group_size, dst, scales);
}

int sdxlq_pack_weight_fp8(sdxlq_context* ctx, const void* src, int32_t src_dtype, uint64_t n, uint64_t k,
                          int32_t fmt, int32_t scale_mode, int32_t layout, uint8_t* dst, float* scales) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    if (src == nullptr || dst == nullptr || scales == nullptr) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "pack_weight_fp8: null pointer");
    if (!is_fp8(fmt)) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "CUDA weight upload target must be FP8");
    if (scale_mode != SDXLQ_SCALE_TENSOR_WIDE && scale_mode != SDXLQ_SCALE_PER_OUTPUT_CHANNEL) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "per-output-channel FP8 scaling requires a rank-2 matrix");
    }
    if (n == 0 || k == 0 || n > 0x7FFFFFFFull || k > 0x7FFFFFFFull) return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "pack_weight_fp8: bad shape");
    if (src_dtype != SDXLQ_FP16 && src_dtype != SDXLQ_FP32 && !is_fp8(src_dtype)) {
        return fail(ctx, SDXLQ_ERR_INVALID_ARGUMENT, "pack_weight_fp8: unsupported source type");
    }
    const uint32_t per_channel = scale_mode == SDXLQ_SCALE_PER_OUTPUT_CHANNEL ? 1 : 0;
    const uint32_t scale_count = per_channel ? static_cast<uint32_t>(n) : 1;
    if (src_dtype == fmt && layout == SDXLQ_ROW_MAJOR_NK) {
        // Native FP8 checkpoint: bytes are kept, scales are 1 (weights.cu:331-347).
        cudaError_t error = cudaMemcpyAsync(dst, src, n * k, cudaMemcpyDeviceToDevice, ctx->stream);
        if (error == cudaSuccess) error = launch_fill_f32(scales, scale_count, 1.0f, ctx->stream);
        if (error != cudaSuccess) return fail_cuda(ctx, error, "native FP8 weight copy");
        return SDXLQ_OK;
    }
    const cudaError_t error = launch_fp8_weight_pack(src, src_dtype, static_cast<uint32_t>(n), static_cast<uint32_t>(k),
                                                     fmt == SDXLQ_FP8_E4M3 ? 0 : 1, per_channel,
                                                     layout == SDXLQ_K_MAJOR_KN ? 1 : 0, dst, scales, ctx->stream);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "FP8 weight pack launch");
    return SDXLQ_OK;
}

#ifdef SDXLQ_DIAGNOSTICS
// Tuning build: the 64 control words (error word, then the GEMM kernel's cycle counters of its last launch).
int sdxlq_debug_read_control(sdxlq_context* ctx, uint32_t* out) {
    if (ctx == nullptr || out == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    cudaStreamSynchronize(ctx->stream);
    return cudaMemcpy(out, ctx->control, 64 * sizeof(uint32_t), cudaMemcpyDeviceToHost) == cudaSuccess ? SDXLQ_OK : SDXLQ_ERR_CUDA;
}
#endif

int sdxlq_profile_enable(sdxlq_context* ctx, int enabled) {
    if (ctx == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    ctx->profiling = enabled != 0;
    return SDXLQ_OK;
}

int sdxlq_profile_read(sdxlq_context* ctx, sdxlq_kernel_times* out) {
    if (ctx == nullptr || out == nullptr) return SDXLQ_ERR_INVALID_ARGUMENT;
    const cudaError_t status = cudaStreamSynchronize(ctx->stream);
    if (status != cudaSuccess) return fail_cuda(ctx, status, "stream synchronize");
    std::memset(out, 0, sizeof(*out));
    for (auto& entry : ctx->timed) {
        float milliseconds = 0.0f;
        if (cudaEventElapsedTime(&milliseconds, entry.start, entry.stop) == cudaSuccess &&
            entry.kernel_class >= 0 && entry.kernel_class < SDXLQ_KERNEL_CLASSES) {
            out->milliseconds[entry.kernel_class] += milliseconds;
            out->launches[entry.kernel_class] += static_cast<uint64_t>(entry.launches);
        }
        ctx->event_pool.emplace_back(entry.start, entry.stop);
    }
    ctx->timed.clear();
    return SDXLQ_OK;
}

// Launches a one-thread kernel that waits, with the given limit, on a barrier nothing ever
// signals. The wait runs out, the kernel records the timeout code and returns; the next
// sdxlq_context_check reports SDXLQ_ERR_TIMEOUT and the context stays usable.
int sdxlq_selftest_bounded_wait(sdxlq_context* ctx, long long limit_cycles) {
    if (ctx == nullptr || limit_cycles <= 0 || limit_cycles > 2000000000LL) return SDXLQ_ERR_INVALID_ARGUMENT;
    const cudaError_t error = launch_bounded_wait_probe(ctx->control, limit_cycles, ctx->stream);
    if (error != cudaSuccess) return fail_cuda(ctx, error, "bounded wait probe launch");
    return SDXLQ_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Allocation-free Linear
// ------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;     // quantised-activation scratch, per GPU
constexpr int kStaticMaxDevices = 16;

// Scratch for the quantised activations and the control words (timeout flag, FP8 amax words) of
// the allocation-free entry point. File-scope device arrays: every GPU that loads this library
// holds them until the process exits. Zero-initialised when the module is loaded.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) uint32_t g_static_control[64 + 2 * kMaxFp8Jobs];

struct StaticSlot {
    bool ready = false;
    sdxlq_context context;
};

StaticSlot g_static_slots[kStaticMaxDevices];
std::mutex g_static_mutex;

void copy_message(char* destination, size_t capacity, const std::string& text) {
    if (destination == nullptr || capacity == 0) return;
    const size_t length = std::min(capacity - 1, text.size());
    std::memcpy(destination, text.data(), length);
    destination[length] = '\0';
}

}  // namespace

extern "C" int sdxlq_linear_static(int device, void* stream, const sdxlq_linear_desc* desc, char* message,
                                   size_t message_capacity) {
    copy_message(message, message_capacity, "");
    if (desc == nullptr || device < 0 || device >= kStaticMaxDevices) {
        copy_message(message, message_capacity, "sdxlq_linear_static: null descriptor or device index out of range");
        return SDXLQ_ERR_INVALID_ARGUMENT;
    }
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess || current != device) {
        copy_message(message, message_capacity, "sdxlq_linear_static: `device` must be the calling thread's current CUDA device");
        return SDXLQ_ERR_INVALID_ARGUMENT;
    }
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticSlot& slot = g_static_slots[device];
    if (!slot.ready) {
        // Once per device, with that device current: the array names above are host-side handles,
        // not device addresses; the kernels need the addresses cudaGetSymbolAddress returns.
        void* scratch = nullptr;
        void* control = nullptr;
        cudaError_t status = cudaGetSymbolAddress(&scratch, g_static_scratch);
        if (status == cudaSuccess) status = cudaGetSymbolAddress(&control, g_static_control);
        cudaDeviceProp properties{};
        if (status == cudaSuccess) status = cudaGetDeviceProperties(&properties, device);
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult query{};
        if (status == cudaSuccess) status = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query);
        if (status != cudaSuccess || scratch == nullptr || control == nullptr || entry == nullptr) {
            copy_message(message, message_capacity,
                         std::string("sdxlq_linear_static: set-up failed: ") + cudaGetErrorString(status));
            return SDXLQ_ERR_CUDA;
        }
        if (properties.major != 10) {
            copy_message(message, message_capacity, "sdxlq_linear_static: the kernels are built for sm_100a only");
            return SDXLQ_ERR_UNSUPPORTED_SHAPE;
        }
        slot.context.device = device;
        slot.context.sm_count = properties.multiProcessorCount;
        slot.context.workspace = static_cast<uint8_t*>(scratch);
        slot.context.workspace_bytes = kStaticScratchBytes;
        slot.context.control = static_cast<uint32_t*>(control);
        slot.context.encode = reinterpret_cast<EncodeTiledFn>(entry);
        slot.ready = true;
    }
    const size_t needed = sdxlq_workspace_bytes(desc, 1);
    if (needed > kStaticScratchBytes) {
        char text[192];
        std::snprintf(text, sizeof(text),
                      "sdxlq_linear_static: this projection needs %zu bytes of scratch for its quantised activations, "
                      "the static array holds %zu; use sdxlq_linear with a context instead",
                      needed, kStaticScratchBytes);
        copy_message(message, message_capacity, text);
        return SDXLQ_ERR_WORKSPACE;
    }
    slot.context.stream = static_cast<cudaStream_t>(stream);
    const int result = sdxlq_linear(&slot.context, desc);
    if (result != SDXLQ_OK) copy_message(message, message_capacity, slot.context.last_error);
    return result;
}
