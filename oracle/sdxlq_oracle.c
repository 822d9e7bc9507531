/*
 * TEST INFRASTRUCTURE ONLY. CPU restatement ("oracle") of the arithmetic of the
 * reference project's quantized-Linear path. Nothing in the shipped library may
 * include, link or call this file: it exists to check the CUDA kernels.
 *
 * Parity pin: validated against (1) the reference's own known-answer tests for this
 * path, replayed in tests/test_oracle_golden.py (tests/cuda/cuda_ops_test.cu:187-348
 * of the reference), and (2) the unmodified reference CPU `linear_2d`/`geglu`
 * compiled from the reference sources (oracle/ref_harness_unet.cpp) for the dense
 * path. The quantized arithmetic (INT8 ConvRot, FP8 activations) has no CPU
 * implementation in the reference, so it is restated here line by line from the CUDA
 * sources cited at each function; divisions and reciprocals are IEEE round-to-nearest
 * (the reference's default build uses --use_fast_math, whose approximate division
 * cannot be restated on a CPU). (3) The FP8 activation quantiser, the native FP8 and
 * FP16 projections with their epilogues and LayerNorm are additionally checked on the
 * GPU against the reference's own CUDA translation units compiled for sm_100
 * (oracle/ref_harness_cuda.cpp, tests/test_reference_device_gpu.py).
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -pthread -shared).
 */

#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* ------------------------------------------------------------------------- */
/* Row-parallel helper (plain pthreads; each row is computed by exactly one   */
/* thread with the same scalar code, so results do not depend on the count).  */
/* ------------------------------------------------------------------------- */

typedef void (*row_fn)(size_t row, void* context);

typedef struct {
    row_fn function;
    void* context;
    size_t begin;
    size_t end;
} row_task;

static void* row_worker(void* argument) {
    row_task* task = (row_task*)argument;
    for (size_t row = task->begin; row < task->end; ++row) task->function(row, task->context);
    return NULL;
}

static int g_threads = 0;

int orc_threads(void) {
    if (g_threads <= 0) {
        long detected = sysconf(_SC_NPROCESSORS_ONLN);
        if (detected < 1) detected = 1;
        if (detected > 64) detected = 64;
        g_threads = (int)detected;
    }
    return g_threads;
}

void orc_set_threads(int count) { g_threads = count < 1 ? 1 : (count > 64 ? 64 : count); }

static void parallel_rows(size_t rows, row_fn function, void* context) {
    size_t workers = (size_t)orc_threads();
    if (workers > rows) workers = rows;
    if (workers <= 1) {
        for (size_t row = 0; row < rows; ++row) function(row, context);
        return;
    }
    pthread_t handles[64];
    row_task tasks[64];
    const size_t chunk = (rows + workers - 1) / workers;
    size_t started = 0;
    for (size_t w = 0; w < workers; ++w) {
        tasks[w].function = function;
        tasks[w].context = context;
        tasks[w].begin = w * chunk < rows ? w * chunk : rows;
        tasks[w].end = (w + 1) * chunk < rows ? (w + 1) * chunk : rows;
        if (pthread_create(&handles[w], NULL, row_worker, &tasks[w]) != 0) {
            row_worker(&tasks[w]);
            handles[w] = 0;
            continue;
        }
        ++started;
    }
    (void)started;
    for (size_t w = 0; w < workers; ++w) {
        if (handles[w] != 0) pthread_join(handles[w], NULL);
    }
}

/* ------------------------------------------------------------------------- */
/* Scalar conversions                                                         */
/* ------------------------------------------------------------------------- */

static inline uint32_t f32_bits(float v) { uint32_t b; memcpy(&b, &v, 4); return b; }
static inline float bits_f32(uint32_t b) { float v; memcpy(&v, &b, 4); return v; }

/* IEEE binary16 -> binary32 (exact). Mirrors TensorReader::half_to_float,
 * src/unet.cpp:62-87 of the reference. */
float orc_h2f(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exponent = (h >> 10) & 0x1Fu;
    uint32_t mantissa = h & 0x03FFu;
    if (exponent == 0) {
        if (mantissa == 0) return bits_f32(sign);
        int e = -14;
        while ((mantissa & 0x0400u) == 0) { mantissa <<= 1; --e; }
        mantissa &= 0x03FFu;
        return bits_f32(sign | ((uint32_t)(e + 127) << 23) | (mantissa << 13));
    }
    if (exponent == 0x1Fu) return bits_f32(sign | 0x7F800000u | (mantissa << 13));
    return bits_f32(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

/* binary32 -> binary16, round-to-nearest-even: the semantics of __float2half_rn used by
 * every FP16 store on the path (e.g. src/cuda/int8_convrot.cu:401). */
uint16_t orc_f2h(float value) {
    const uint32_t bits = f32_bits(value);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    const uint32_t absolute = bits & 0x7FFFFFFFu;
    if (absolute > 0x7F800000u) return (uint16_t)(sign | 0x7FFFu);          /* NaN */
    if (absolute >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);         /* >= 65520 -> inf */
    if (absolute < 0x33000001u) return sign;                                /* <= 2^-25 -> 0 */
    const int exponent = (int)(absolute >> 23) - 127;
    uint32_t mantissa = (absolute & 0x007FFFFFu) | 0x00800000u;
    int shift;
    int half_exponent;
    if (exponent < -14) {           /* subnormal half */
        shift = 13 + (-14 - exponent);
        half_exponent = 0;
    } else {
        shift = 13;
        half_exponent = exponent + 15;
    }
    const uint32_t kept = mantissa >> shift;
    const uint32_t remainder = mantissa & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    uint32_t rounded = kept;
    if (remainder > halfway || (remainder == halfway && (kept & 1u))) rounded += 1;
    uint32_t result;
    if (half_exponent == 0) {
        result = rounded;            /* may carry into the exponent: correct by construction */
    } else {
        result = ((uint32_t)half_exponent << 10) + (rounded - 0x0400u);
    }
    return (uint16_t)(sign | result);
}

/* FP8 byte -> float. fmt 0 = E4M3FN (bias 7, no inf, 0x7F/0xFF NaN), fmt 1 = E5M2 (bias 15,
 * IEEE inf/NaN). Mirrors TensorReader::fp8_to_float, src/unet.cpp:93-119, and the device
 * decoder in src/cuda/tensor.cu:78-110 of the reference. */
float orc_fp8_decode(uint8_t bits, int fmt) {
    const int exponent_bits = fmt == 0 ? 4 : 5;
    const int mantissa_bits = fmt == 0 ? 3 : 2;
    const int bias = fmt == 0 ? 7 : 15;
    const int negative = (bits & 0x80u) != 0;
    const unsigned exponent_mask = (1u << exponent_bits) - 1u;
    const unsigned mantissa_mask = (1u << mantissa_bits) - 1u;
    const unsigned exponent = (bits >> mantissa_bits) & exponent_mask;
    const unsigned mantissa = bits & mantissa_mask;
    float value = 0.0f;
    if (exponent == 0) {
        if (mantissa != 0) value = ldexpf((float)mantissa / (float)(1u << mantissa_bits), 1 - bias);
    } else if (fmt == 1 && exponent == exponent_mask) {
        value = mantissa == 0 ? INFINITY : NAN;
    } else if (fmt == 0 && exponent == exponent_mask && mantissa == mantissa_mask) {
        value = NAN;
    } else {
        value = ldexpf(1.0f + (float)mantissa / (float)(1u << mantissa_bits), (int)exponent - bias);
    }
    return negative ? -value : value;
}

/* float -> FP8 byte with round-to-nearest-even and saturation to the largest finite value:
 * the semantics of the `__nv_fp8_e4m3(float)` / `__nv_fp8_e5m2(float)` constructors used at
 * src/cuda/fp8_kernels.cu:48 and src/cuda/weights.cu:170 of the reference
 * (cvt.rn.satfinite). NaN maps to 0x7F. */
uint8_t orc_fp8_encode(float value, int fmt) {
    const int mantissa_bits = fmt == 0 ? 3 : 2;
    const int bias = fmt == 0 ? 7 : 15;
    const int min_normal_exponent = 1 - bias;
    const float maximum = fmt == 0 ? 448.0f : 57344.0f;
    const uint8_t max_bits = fmt == 0 ? 0x7Eu : 0x7Bu;
    const uint8_t sign = (f32_bits(value) >> 31) ? 0x80u : 0x00u;
    if (isnan(value)) return (uint8_t)(sign | 0x7Fu);
    const double magnitude = fabs((double)value);
    if (magnitude >= (double)maximum) return (uint8_t)(sign | max_bits);
    if (magnitude == 0.0) return sign;
    int exponent;
    (void)frexp(magnitude, &exponent);      /* magnitude = f * 2^exponent, f in [0.5,1) */
    exponent -= 1;                          /* floor(log2(magnitude)) */
    if (exponent < min_normal_exponent) exponent = min_normal_exponent;
    const double quantum = ldexp(1.0, exponent - mantissa_bits);
    const double steps = nearbyint(magnitude / quantum);     /* RNE under the default mode */
    double rounded = steps * quantum;
    if (rounded > (double)maximum) return (uint8_t)(sign | max_bits);
    if (rounded == 0.0) return sign;
    int rounded_exponent;
    (void)frexp(rounded, &rounded_exponent);
    rounded_exponent -= 1;
    uint8_t encoded;
    if (rounded_exponent < min_normal_exponent) {
        const unsigned mantissa = (unsigned)(rounded / ldexp(1.0, min_normal_exponent - mantissa_bits));
        encoded = (uint8_t)mantissa;
    } else {
        const double fraction = rounded / ldexp(1.0, rounded_exponent) - 1.0;
        const unsigned mantissa = (unsigned)(fraction * (double)(1u << mantissa_bits));
        encoded = (uint8_t)((((unsigned)(rounded_exponent + bias)) << mantissa_bits) | mantissa);
    }
    return (uint8_t)(sign | encoded);
}

void orc_h2f_array(const uint16_t* in, float* out, size_t count) {
    for (size_t i = 0; i < count; ++i) out[i] = orc_h2f(in[i]);
}

void orc_f2h_array(const float* in, uint16_t* out, size_t count) {
    for (size_t i = 0; i < count; ++i) out[i] = orc_f2h(in[i]);
}

void orc_fp8_decode_array(const uint8_t* in, float* out, size_t count, int fmt) {
    for (size_t i = 0; i < count; ++i) out[i] = orc_fp8_decode(in[i], fmt);
}

void orc_fp8_encode_array(const float* in, uint8_t* out, size_t count, int fmt) {
    for (size_t i = 0; i < count; ++i) out[i] = orc_fp8_encode(in[i], fmt);
}

/* ------------------------------------------------------------------------- */
/* INT8 ConvRot                                                               */
/* ------------------------------------------------------------------------- */

/* bool valid_convrot_group_size(size_t): src/cuda/int8_convrot.cu:489-496. */
int orc_valid_convrot_group_size(size_t group_size) {
    if (group_size < 4 || group_size > 256) return 0;
    while (group_size > 1) {
        if (group_size % 4 != 0) return 0;
        group_size /= 4;
    }
    return 1;
}

/* regular_hadamard_transform: src/cuda/int8_convrot.cu:121-150. Radix-4 butterflies with
 * stride 1, 4, 16, 64; element `index` of a stage takes the 4-tuple (a,b,c,d) spaced by
 * `stride` inside its block of 4*stride and combines it by its position in the tuple, with
 * the additions evaluated left to right exactly as written in the reference.
 * `primary` holds the input; the result is in the returned buffer. */
static float* hadamard_group(float* primary, float* scratch, size_t group_size) {
    float* source = primary;
    float* destination = scratch;
    for (size_t stride = 1; stride < group_size; stride *= 4) {
        for (size_t index = 0; index < group_size; ++index) {
            const size_t block = index / (4 * stride);
            const size_t offset = index % stride;
            const size_t lane = (index / stride) % 4;
            const size_t base = block * 4 * stride + offset;
            const float a = source[base];
            const float b = source[base + stride];
            const float c = source[base + 2 * stride];
            const float d = source[base + 3 * stride];
            float value;
            if (lane == 0) value = a + b + c - d;
            else if (lane == 1) value = a + b - c + d;
            else if (lane == 2) value = a - b + c + d;
            else value = -a + b + c + d;
            destination[index] = value;
        }
        float* swap = source; source = destination; destination = swap;
    }
    return source;
}

void orc_hadamard_rows(const float* input, float* output, size_t rows, size_t columns, size_t group_size) {
    float primary[256], scratch[256];
    for (size_t row = 0; row < rows; ++row) {
        for (size_t group = 0; group < columns; group += group_size) {
            memcpy(primary, input + row * columns + group, group_size * sizeof(float));
            const float* transformed = hadamard_group(primary, scratch, group_size);
            memcpy(output + row * columns + group, transformed, group_size * sizeof(float));
        }
    }
}

/* __float2int_rn followed by the clamp of src/cuda/int8_convrot.cu:222-225 / 325-329. */
static inline int8_t quantize_value(float scaled) {
    int quantized;
    if (isnan(scaled)) quantized = 0;
    else if (scaled >= 2147483648.0f) quantized = 2147483647;
    else if (scaled <= -2147483648.0f) quantized = (-2147483647 - 1);
    else quantized = (int)nearbyintf(scaled);
    if (quantized < -128) quantized = -128;
    if (quantized > 127) quantized = 127;
    return (int8_t)quantized;
}

/* Row-wise rotate + scale + quantize. The weight path (weight_amax_kernel /
 * quantize_weight_kernel, src/cuda/int8_convrot.cu:156-249) and the activation path
 * (activation_amax_kernel / quantize_activation_kernel, :265-353) use the same arithmetic:
 *   rotated = hadamard(group) * g^-1/2       (g == 0: no rotation, no normalisation)
 *   amax    = max over finite |rotated|
 *   scale   = amax > 0 ? max(amax / 127, 1e-30) : 1
 *   q       = clamp(rn(rotated * (1 / scale)), -128, 127)
 * `input` holds the FP32 value of each element (FP16 sources are widened exactly first). */
typedef struct {
    const float* input; size_t columns; size_t group_size; int8_t* quantized; float* scales;
} quantize_rows_ctx;

static void quantize_row(size_t row, void* context) {
    const quantize_rows_ctx* c = (const quantize_rows_ctx*)context;
    const size_t columns = c->columns, group_size = c->group_size;
    const float* source = c->input + row * columns;
    int8_t* destination = c->quantized + row * columns;
    float primary[256], scratch[256];
    float maximum = 0.0f;
    /* rsqrtf(g) for g in {4,16,64,256} is the exact power of two 2^-k. */
    const float normalization = group_size ? 1.0f / sqrtf((float)group_size) : 1.0f;
    if (group_size == 0) {
        for (size_t column = 0; column < columns; ++column) {
            const float value = fabsf(source[column]);
            if (isfinite(value) && value > maximum) maximum = value;
        }
    } else {
        for (size_t group = 0; group < columns; group += group_size) {
            memcpy(primary, source + group, group_size * sizeof(float));
            const float* transformed = hadamard_group(primary, scratch, group_size);
            for (size_t i = 0; i < group_size; ++i) {
                const float value = fabsf(transformed[i] * normalization);
                if (isfinite(value) && value > maximum) maximum = value;
            }
        }
    }
    const float scale = maximum > 0.0f ? fmaxf(maximum / 127.0f, 1.0e-30f) : 1.0f;
    c->scales[row] = scale;
    const float inverse_scale = 1.0f / scale;
    if (group_size == 0) {
        for (size_t column = 0; column < columns; ++column) {
            destination[column] = quantize_value(source[column] * inverse_scale);
        }
    } else {
        for (size_t group = 0; group < columns; group += group_size) {
            memcpy(primary, source + group, group_size * sizeof(float));
            const float* transformed = hadamard_group(primary, scratch, group_size);
            for (size_t i = 0; i < group_size; ++i) {
                destination[group + i] = quantize_value(transformed[i] * normalization * inverse_scale);
            }
        }
    }
}

void orc_int8_quantize_rows(const float* input, size_t rows, size_t columns, size_t group_size,
                            int8_t* quantized, float* scales) {
    quantize_rows_ctx c = {input, columns, group_size, quantized, scales};
    parallel_rows(rows, quantize_row, &c);
}

/* Integer GEMM ACC[M,N] = Xq[M,K] * Wq[N,K]^T: the contract of the cuBLASLt COMPUTE_32I call
 * (src/cuda/int8_convrot.cu:404-447, 684-691) and of int8_gemm_dp4a_kernel (:355-371).
 * Integer arithmetic: any summation order gives the same result. */
typedef struct {
    const int8_t* activations; const int8_t* weights; int32_t* accumulator;
    size_t output_columns; size_t inner;
} int8_gemm_ctx;

static void int8_gemm_row(size_t row, void* context) {
    const int8_gemm_ctx* c = (const int8_gemm_ctx*)context;
    const int8_t* a = c->activations + row * c->inner;
    for (size_t column = 0; column < c->output_columns; ++column) {
        const int8_t* w = c->weights + column * c->inner;
        int32_t sum = 0;
        for (size_t i = 0; i < c->inner; ++i) sum += (int32_t)a[i] * (int32_t)w[i];
        c->accumulator[row * c->output_columns + column] = sum;
    }
}

void orc_int8_gemm_i32(const int8_t* activations, const int8_t* weights, int32_t* accumulator,
                       size_t rows, size_t output_columns, size_t inner) {
    int8_gemm_ctx c = {activations, weights, accumulator, output_columns, inner};
    parallel_rows(rows, int8_gemm_row, &c);
}

/* dequantize_gemm_f16_kernel: src/cuda/int8_convrot.cu:388-402.
 * out = half_rn((float(acc) * a_scale[row]) * w_scale[col]). */
typedef struct {
    const int32_t* accumulator; const float* activation_scales; const float* weight_scales;
    size_t columns; uint16_t* output;
} dequant_ctx;

static void dequant_row(size_t row, void* context) {
    const dequant_ctx* c = (const dequant_ctx*)context;
    for (size_t column = 0; column < c->columns; ++column) {
        const size_t index = row * c->columns + column;
        const float value = (float)c->accumulator[index] * c->activation_scales[row] * c->weight_scales[column];
        c->output[index] = orc_f2h(value);
    }
}

void orc_int8_dequant_f16(const int32_t* accumulator, const float* activation_scales,
                          const float* weight_scales, size_t rows, size_t columns, uint16_t* output) {
    dequant_ctx c = {accumulator, activation_scales, weight_scales, columns, output};
    parallel_rows(rows, dequant_row, &c);
}

/* ------------------------------------------------------------------------- */
/* Epilogues                                                                  */
/* ------------------------------------------------------------------------- */

/* apply_linear_activation: src/cuda/ops_kernels.cu:128-140. 1=SiLU 2=GELU(erf) 3=QuickGELU. */
static inline float apply_activation(float x, int activation) {
    if (activation == 1) return x / (1.0f + expf(-x));
    if (activation == 2) return 0.5f * x * (1.0f + erff(x * 0.7071067811865475f));
    if (activation == 3) return x / (1.0f + expf(-1.702f * x));
    return x;
}

typedef struct {
    uint16_t* values; const uint16_t* bias; size_t width; int activation;
    const uint16_t* projected; uint16_t* output;
} epilogue_ctx;

/* add_last_dim_bias_kernel: src/cuda/ops_kernels.cu:76-82 — `__hadd` of two halves. The
 * exact sum rounded once to half equals half_rn(float(a) + float(b)) because binary32 keeps
 * at least 2*11+2 significand bits. */
static void bias_add_row(size_t row, void* context) {
    const epilogue_ctx* c = (const epilogue_ctx*)context;
    for (size_t column = 0; column < c->width; ++column) {
        const size_t index = row * c->width + column;
        c->values[index] = orc_f2h(orc_h2f(c->values[index]) + orc_h2f(c->bias[column]));
    }
}

void orc_bias_add_f16(uint16_t* values, const uint16_t* bias, size_t rows, size_t width) {
    epilogue_ctx c = {values, bias, width, 0, NULL, NULL};
    parallel_rows(rows, bias_add_row, &c);
}

/* bias_activation_in_place_kernel: src/cuda/ops_kernels.cu:142-153. */
static void bias_activation_row(size_t row, void* context) {
    const epilogue_ctx* c = (const epilogue_ctx*)context;
    for (size_t column = 0; column < c->width; ++column) {
        const size_t index = row * c->width + column;
        const float x = orc_h2f(c->values[index]) + orc_h2f(c->bias[column]);
        c->values[index] = orc_f2h(apply_activation(x, c->activation));
    }
}

void orc_bias_activation_f16(uint16_t* values, const uint16_t* bias, size_t rows, size_t width,
                             int activation) {
    epilogue_ctx c = {values, bias, width, activation, NULL, NULL};
    parallel_rows(rows, bias_activation_row, &c);
}

/* bias_geglu_kernel: src/cuda/ops_kernels.cu:167-183. `projected` is [rows, 2*width]; the
 * first half of each row is the value, the second half the gate. */
static void bias_geglu_row(size_t row, void* context) {
    const epilogue_ctx* c = (const epilogue_ctx*)context;
    const size_t width = c->width;
    const size_t base = row * width * 2;
    for (size_t column = 0; column < width; ++column) {
        const float value = orc_h2f(c->projected[base + column]) + orc_h2f(c->bias[column]);
        const float gate = orc_h2f(c->projected[base + width + column]) + orc_h2f(c->bias[width + column]);
        const float gelu = 0.5f * gate * (1.0f + erff(gate * 0.7071067811865475f));
        c->output[row * width + column] = orc_f2h(value * gelu);
    }
}

void orc_bias_geglu_f16(const uint16_t* projected, const uint16_t* bias, uint16_t* output,
                        size_t rows, size_t width) {
    epilogue_ctx c = {NULL, bias, width, 4, projected, output};
    parallel_rows(rows, bias_geglu_row, &c);
}

/* ------------------------------------------------------------------------- */
/* FP8                                                                        */
/* ------------------------------------------------------------------------- */

/* quantize_tensor_fp8: src/cuda/fp8_kernels.cu:16-49, 157-190. Tensor-wide dynamic scale:
 *   amax = max |x| (x widened from half), scale = amax > 0 ? max(amax / FP8_MAX, 1e-12) : 1
 *   q = FP8_satfinite(x * (1 / scale)).  Returns the dequantisation scale. */
float orc_fp8_quantize_activation(const uint16_t* source, size_t count, int fmt, uint8_t* destination) {
    float maximum = 0.0f;
    for (size_t i = 0; i < count; ++i) maximum = fmaxf(maximum, fabsf(orc_h2f(source[i])));
    const float fp8_maximum = fmt == 0 ? 448.0f : 57344.0f;
    const float scale = maximum > 0.0f ? fmaxf(maximum / fp8_maximum, 1.0e-12f) : 1.0f;
    const float inverse_scale = 1.0f / scale;
    for (size_t i = 0; i < count; ++i) {
        destination[i] = orc_fp8_encode(orc_h2f(source[i]) * inverse_scale, fmt);
    }
    return scale;
}

/* Load-time FP8 weight quantisation: source_amax_kernel / finalize_fp8_scales_kernel /
 * pack_to_fp8_kernel, src/cuda/weights.cu:119-170. scale_count is 1 (tensor-wide) or `rows`
 * (per output channel); non-finite values are skipped by the amax; q = FP8(value / scale).
 * k_major != 0 stores the transposed [columns, rows] layout (FP8StorageLayout::KMajorKN). */
void orc_fp8_quantize_weight(const float* source, size_t rows, size_t columns, int fmt,
                             size_t scale_count, int k_major, uint8_t* destination, float* scales) {
    const float fp8_maximum = fmt == 0 ? 448.0f : 57344.0f;
    for (size_t s = 0; s < scale_count; ++s) scales[s] = 0.0f;
    for (size_t row = 0; row < rows; ++row) {
        for (size_t column = 0; column < columns; ++column) {
            const float value = fabsf(source[row * columns + column]);
            if (!isfinite(value)) continue;
            const size_t s = scale_count == 1 ? 0 : row;
            if (value > scales[s]) scales[s] = value;
        }
    }
    for (size_t s = 0; s < scale_count; ++s) {
        scales[s] = scales[s] > 0.0f ? fmaxf(scales[s] / fp8_maximum, 1.0e-12f) : 1.0f;
    }
    for (size_t row = 0; row < rows; ++row) {
        const float scale = scales[scale_count == 1 ? 0 : row];
        for (size_t column = 0; column < columns; ++column) {
            const size_t index = k_major ? column * rows + row : row * columns + column;
            destination[index] = orc_fp8_encode(source[row * columns + column] / scale, fmt);
        }
    }
}

/* Native FP8 Linear contract (native_fp8_linear, src/cuda/ops_blas.cpp:153-225):
 *   Y[m,n] = half((sum_k fp8(x[m,k]) * fp8(w[n,k])) * x_scale * w_scale[n or 0]).
 * The reference leaves the summation order to cuBLASLt; the oracle accumulates the exact
 * products in binary64 and rounds once to binary32, so it is the order-free target value. */
typedef struct {
    const uint8_t* activations; const uint8_t* weights; const float* activation_lut;
    const float* weight_lut; float activation_scale; const float* weight_scales;
    size_t weight_scale_count; size_t output_columns; size_t inner; uint16_t* output;
    float* accumulator_out;
} fp8_linear_ctx;

static void fp8_linear_row(size_t row, void* context) {
    const fp8_linear_ctx* c = (const fp8_linear_ctx*)context;
    const uint8_t* a = c->activations + row * c->inner;
    for (size_t column = 0; column < c->output_columns; ++column) {
        const uint8_t* w = c->weights + column * c->inner;
        double sum = 0.0;
        for (size_t i = 0; i < c->inner; ++i) sum += (double)c->activation_lut[a[i]] * (double)c->weight_lut[w[i]];
        const float accumulator = (float)sum;
        const size_t index = row * c->output_columns + column;
        if (c->accumulator_out != NULL) c->accumulator_out[index] = accumulator;
        const float scale = c->weight_scales[c->weight_scale_count == 1 ? 0 : column];
        c->output[index] = orc_f2h(accumulator * c->activation_scale * scale);
    }
}

void orc_fp8_linear_f16(const uint8_t* activations, int activation_fmt, float activation_scale,
                        const uint8_t* weights, int weight_fmt, const float* weight_scales,
                        size_t weight_scale_count, size_t rows, size_t output_columns, size_t inner,
                        uint16_t* output, float* accumulator_out) {
    float activation_lut[256], weight_lut[256];
    for (int i = 0; i < 256; ++i) {
        activation_lut[i] = orc_fp8_decode((uint8_t)i, activation_fmt);
        weight_lut[i] = orc_fp8_decode((uint8_t)i, weight_fmt);
    }
    fp8_linear_ctx c = {activations, weights, activation_lut, weight_lut, activation_scale,
                        weight_scales, weight_scale_count, output_columns, inner, output,
                        accumulator_out};
    parallel_rows(rows, fp8_linear_row, &c);
}

/* ------------------------------------------------------------------------- */
/* Dense path                                                                 */
/* ------------------------------------------------------------------------- */

/* linear_2d: src/unet.cpp:202-225 — FP32 accumulator initialised with the bias, products
 * added in index order, no fused multiply-add. `weights` holds FP32 values (weights stored as
 * F16/FP8 are widened exactly by the caller, as TensorReader::read does). */
typedef struct {
    const float* input; const float* weights; const float* bias;
    size_t output_columns; size_t inner; float* output;
} linear_ctx;

static void linear_row(size_t row, void* context) {
    const linear_ctx* c = (const linear_ctx*)context;
    const float* source = c->input + row * c->inner;
    for (size_t column = 0; column < c->output_columns; ++column) {
        const float* w = c->weights + column * c->inner;
        float value = c->bias != NULL ? c->bias[column] : 0.0f;
        for (size_t i = 0; i < c->inner; ++i) value += source[i] * w[i];
        c->output[row * c->output_columns + column] = value;
    }
}

void orc_linear_f32(const float* input, const float* weights, const float* bias,
                    size_t rows, size_t output_columns, size_t inner, float* output) {
    linear_ctx c = {input, weights, bias, output_columns, inner, output};
    parallel_rows(rows, linear_row, &c);
}

/* geglu + gelu: src/unet.cpp:190-193, 483-493 (FP32, exact-erf GELU on the second half). */
void orc_geglu_f32(const float* input, size_t rows, size_t width, float* output) {
    for (size_t row = 0; row < rows; ++row) {
        const float* source = input + row * width * 2;
        for (size_t column = 0; column < width; ++column) {
            const float gate = source[width + column];
            output[row * width + column] =
                source[column] * (0.5f * gate * (1.0f + erff(gate * 0.7071067811865475244f)));
        }
    }
}

/* layer_norm_kernel (src/cuda/ops_kernels.cu:185-221): per row, FP32 sum -> mean, FP32 sum of the
 * centred squares -> variance clamped at 0, inverse = 1 / sqrt(variance + epsilon), output =
 * half_rn((x - mean) * inverse * gamma + beta) with the last multiply-add fused as nvcc contracts
 * it. The reference adds the partial sums of 256 threads through a shared-memory tree and takes
 * rsqrtf (2 ulp); here the sums run in column order and the reciprocal square root is the
 * correctly rounded quotient, so results may differ from the device in the last FP32 bits of the
 * statistics. */
void orc_layer_norm_f16(const uint16_t* input, const uint16_t* gamma, const uint16_t* beta, size_t rows,
                        size_t width, float epsilon, uint16_t* output) {
    for (size_t row = 0; row < rows; ++row) {
        const uint16_t* x = input + row * width;
        float sum = 0.0f;
        for (size_t c = 0; c < width; ++c) sum += orc_h2f(x[c]);
        const float mean = sum / (float)width;
        float squares = 0.0f;
        for (size_t c = 0; c < width; ++c) {
            const float centred = orc_h2f(x[c]) - mean;
            squares = fmaf(centred, centred, squares);
        }
        float variance = squares / (float)width;
        if (!(variance > 0.0f)) variance = 0.0f;
        const float inverse = 1.0f / sqrtf(variance + epsilon);
        for (size_t c = 0; c < width; ++c) {
            const float scaled = (orc_h2f(x[c]) - mean) * inverse;
            output[row * width + c] = orc_f2h(fmaf(scaled, orc_h2f(gamma[c]), orc_h2f(beta[c])));
        }
    }
}
