/*
 * nslq_oracle.c -- CPU restatement of the NSL quantized-linear path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against (and the timed CPU baseline of the benchmark).  Nothing in the product
 * library links, loads or calls it.
 *
 * Parity pin: every function below is checked against the golden vectors the
 * NSL tests hold for this path (the ten BitNet forward fixtures, the four
 * absmax-quant fixtures, byte 0x1A / the 81 trit round trips, the loader
 * vector with scale 0.925, the half-away rounding row, the AWQ unit-test
 * constants).  The NSL sources themselves are Rust and cannot be compiled in
 * this environment, so the pin is by golden vector, not by linking the original.
 *
 * Each function names the NSL file:line it restates (paths are relative to the
 * NSL source tree).  Build with:  gcc -O2 -ffp-contract=off -fno-fast-math
 * (contraction off: the Rust reference never fuses a multiply with an add).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* Minimal parallel-for over [0,n): `threads` POSIX threads, static contiguous
 * split.  threads <= 1 runs inline in ascending order. */
typedef void (*nslo_range_fn)(int64_t begin, int64_t end, void *ctx);
typedef struct { nslo_range_fn fn; void *ctx; int64_t b, e; } nslo_job;
static void *nslo_job_main(void *p)
{
    nslo_job *j = (nslo_job *)p;
    j->fn(j->b, j->e, j->ctx);
    return NULL;
}
static void nslo_parallel_for(int64_t n, int threads, nslo_range_fn fn, void *ctx)
{
    if (threads <= 1 || n <= 1) { fn(0, n, ctx); return; }
    if (threads > 256) threads = 256;
    if (threads > n) threads = (int)n;
    pthread_t tid[256];
    nslo_job job[256];
    int64_t per = (n + threads - 1) / threads;
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        int64_t b = t * per, e = b + per < n ? b + per : n;
        if (b >= e) break;
        job[t].fn = fn; job[t].ctx = ctx; job[t].b = b; job[t].e = e;
        if (pthread_create(&tid[t], NULL, nslo_job_main, &job[t]) != 0) {
            fn(b, e, ctx); /* could not spawn: run inline */
            tid[t] = 0;
        }
        started = t + 1;
    }
    for (int t = 0; t < started; ++t)
        if (tid[t]) pthread_join(tid[t], NULL);
}

/* ------------------------------------------------------------------------- */
/* BitLinear: activation quantisation                                         */
/* ------------------------------------------------------------------------- */

/* crates/nsl-codegen/tests/bitnet_reference_impl.rs:46-52  absmax_scale_row.
 * Rust `f32::max` returns the non-NaN operand, which is what fmaxf does. */
float nslo_absmax_scale_row(const float *row, int64_t k)
{
    float acc = 0.0f;
    for (int64_t i = 0; i < k; ++i)
        acc = fmaxf(acc, fabsf(row[i]));
    return acc;
}

/* Rust `as i8` on an f32: saturating, NaN -> 0. */
static inline int8_t sat_i8(float v)
{
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v; /* v is integral here */
}

/* Rust `f32::clamp(min,max)`: NaN passes through. */
static inline float clampf(float v, float lo, float hi)
{
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* crates/nsl-codegen/tests/bitnet_reference_impl.rs:58-70  quantize_row_int8.
 * roundf() rounds half away from zero, as Rust `f32::round` does. */
void nslo_quantize_row_int8(const float *row, int64_t k, float scale, int8_t *q)
{
    if (scale == 0.0f) {
        memset(q, 0, (size_t)k);
        return;
    }
    const float inv_scale = 127.0f / scale;
    for (int64_t i = 0; i < k; ++i) {
        float scaled = row[i] * inv_scale;
        float clipped = clampf(scaled, -127.0f, 127.0f);
        q[i] = sat_i8(roundf(clipped));
    }
}

/* crates/nsl-runtime/src/tensor/mod.rs:3016-3035  nsl_tensor_rmsnorm, f32 input, CPU arm:
 * sequential f64 sum of squares, rms = sqrt(sum/n + eps), out = (f32)(x / rms * w). */
void nslo_rmsnorm_f32(const float *x, const float *w, double eps, int64_t rows, int64_t n, float *out)
{
    for (int64_t r = 0; r < rows; ++r) {
        const float *xr = x + r * n;
        double sum_sq = 0.0;
        for (int64_t j = 0; j < n; ++j) sum_sq += (double)xr[j] * (double)xr[j];
        const double rms = sqrt(sum_sq / (double)n + eps);
        for (int64_t j = 0; j < n; ++j) out[r * n + j] = (float)((double)xr[j] / rms * (double)w[j]);
    }
}

/* crates/nsl-codegen/tests/bitnet_reference_impl.rs:77-95  ternary_gemm_element.
 * Returns the i32 accumulator through *acc_out as well (the bit-exact target). */
float nslo_ternary_gemm_element(const int8_t *q, const int8_t *wcol, int64_t k,
                                float scale, int32_t *acc_out)
{
    int32_t acc = 0;
    for (int64_t i = 0; i < k; ++i)
        acc += (int32_t)q[i] * (int32_t)wcol[i];
    if (acc_out) *acc_out = acc;
    return (scale / 127.0f) * (float)acc;
}

/* crates/nsl-codegen/tests/bitnet_reference_impl.rs:101-141  forward_reference.
 * weights are [hidden][out] row-major trits, exactly as the reference indexes
 * them (column gather per output).  Outputs: scales[rows], q[rows*hidden],
 * acc[rows*out] (may be NULL), y[rows*out]. */
void nslo_forward_reference(const float *acts, int64_t rows, int64_t hidden,
                            const int8_t *weights_kn, int64_t out_dim,
                            float *scales, int8_t *q, int32_t *acc, float *y)
{
    int8_t *col = (int8_t *)malloc((size_t)hidden);
    for (int64_t r = 0; r < rows; ++r) {
        const float *row = acts + r * hidden;
        float scale = nslo_absmax_scale_row(row, hidden);
        int8_t *qr = q + r * hidden;
        nslo_quantize_row_int8(row, hidden, scale, qr);
        for (int64_t c = 0; c < out_dim; ++c) {
            for (int64_t kk = 0; kk < hidden; ++kk)
                col[kk] = weights_kn[kk * out_dim + c];
            int32_t a;
            y[r * out_dim + c] = nslo_ternary_gemm_element(qr, col, hidden, scale, &a);
            if (acc) acc[r * out_dim + c] = a;
        }
        scales[r] = scale;
    }
    free(col);
}

/* ------------------------------------------------------------------------- */
/* BitLinear: 2-bit trit packing                                              */
/* ------------------------------------------------------------------------- */

/* crates/nsl-codegen/src/bitnet/pack.rs:11-19  encode_trit; returns 0xFF for an
 * input outside {-1,0,+1} (the reference panics). */
static inline uint8_t encode_trit(int8_t t)
{
    return (t == -1) ? 0u : (t == 0) ? 1u : (t == 1) ? 2u : 0xFFu;
}

/* crates/nsl-codegen/src/bitnet/pack.rs:38-43  pack_trits, HIGH-BITS-FIRST.
 * Returns -1 on an invalid trit. */
int nslo_pack_trits(const int8_t t[4], uint8_t *byte_out)
{
    uint8_t c0 = encode_trit(t[0]), c1 = encode_trit(t[1]);
    uint8_t c2 = encode_trit(t[2]), c3 = encode_trit(t[3]);
    if ((c0 | c1 | c2 | c3) == 0xFFu) return -1;
    *byte_out = (uint8_t)((c0 << 6) | (c1 << 4) | (c2 << 2) | c3);
    return 0;
}

/* crates/nsl-codegen/src/bitnet/pack.rs:60-67  try_unpack_byte.
 * Returns -1 when any 2-bit field is the reserved 0b11. */
int nslo_try_unpack_byte(uint8_t b, int8_t out[4])
{
    for (int i = 0; i < 4; ++i) {
        uint8_t f = (uint8_t)((b >> (6 - 2 * i)) & 3u);
        if (f == 3u) return -1;
        out[i] = (int8_t)f - 1;
    }
    return 0;
}

/* crates/nsl-codegen/src/bitnet/pack.rs:71-82  pack_trit_slice (n % 4 == 0). */
int nslo_pack_trit_slice(const int8_t *trits, int64_t n, uint8_t *bytes)
{
    if (n % 4 != 0) return -2;
    for (int64_t i = 0; i < n / 4; ++i)
        if (nslo_pack_trits(trits + 4 * i, bytes + i)) return -1;
    return 0;
}

/* crates/nsl-codegen/src/bitnet/pack.rs:87-93  unpack_byte_slice. */
int nslo_unpack_byte_slice(const uint8_t *bytes, int64_t nbytes, int8_t *trits)
{
    for (int64_t i = 0; i < nbytes; ++i)
        if (nslo_try_unpack_byte(bytes[i], trits + 4 * i)) return -1;
    return 0;
}

/* crates/nsl-codegen/src/bitnet/loader.rs:126-193  quantize_float_to_ternary
 * (after widening to f32): absmean scale summed sequentially in f32, round half
 * away, pack.  Returns -2 if numel % 4 != 0 (the reference's AlignmentError). */
int nslo_quantize_float_to_ternary(const float *w, int64_t numel, uint8_t *packed,
                                   int8_t *trits_out, float *scale_out)
{
    if (numel % 4 != 0) return -2;
    float abs_sum = 0.0f;
    for (int64_t i = 0; i < numel; ++i) abs_sum += fabsf(w[i]);
    float scale = abs_sum / (float)numel;
    float eff = scale > 0.0f ? scale : 1.0f;
    for (int64_t i = 0; i < numel; i += 4) {
        int8_t t[4];
        for (int j = 0; j < 4; ++j) {
            float scaled = w[i + j] / eff;
            t[j] = sat_i8(roundf(clampf(scaled, -1.0f, 1.0f)));
            if (trits_out) trits_out[i + j] = t[j];
        }
        if (nslo_pack_trits(t, packed + i / 4)) return -1;
    }
    *scale_out = scale;
    return 0;
}

/* ------------------------------------------------------------------------- */
/* BitLinear forward on the packed kernel layout W[out][hidden/4]             */
/* ------------------------------------------------------------------------- */

typedef struct {
    const float *x; int64_t rows, hidden; const uint8_t *packed; int64_t out_dim;
    float weight_scale; float *scales; int8_t *q; int32_t *acc; float *y; int bad;
} bl_ctx;

static void bl_cols(int64_t c0, int64_t c1, void *p)
{
    bl_ctx *s = (bl_ctx *)p;
    const int64_t hidden = s->hidden, rb = hidden / 4;
    int8_t *wrow = (int8_t *)malloc((size_t)hidden);
    for (int64_t c = c0; c < c1; ++c) {
        if (nslo_unpack_byte_slice(s->packed + c * rb, rb, wrow)) s->bad = 1;
        for (int64_t r = 0; r < s->rows; ++r) {
            const int8_t *qr = s->q + r * hidden;
            int32_t a = 0;
            for (int64_t kk = 0; kk < hidden; ++kk)
                a += (int32_t)qr[kk] * (int32_t)wrow[kk];
            if (s->acc) s->acc[r * s->out_dim + c] = a;
            float v = (s->scales[r] / 127.0f) * (float)a;
            s->y[r * s->out_dim + c] = v * s->weight_scale;
        }
    }
    free(wrow);
}

/* Same arithmetic as forward_reference + the kernel's finalize phase
 * (crates/nsl-codegen/src/bitnet/phases/finalize.rs:39-53: `* weight_scale`
 * as a separately rounded multiply), but with the weight stored the way the
 * reference GPU kernel reads it: row-major [out_dim][hidden_dim] trits packed
 * four per byte along k (crates/nsl-codegen/src/bitnet/mod.rs:97-103).
 * threads <= 1 is the faithful single-thread order; threads > 1 splits the
 * output columns over POSIX threads (our parallelisation; integer sums are exact so
 * the result is identical). */
int nslo_bitlinear_forward_packed(const float *x, int64_t rows, int64_t hidden,
                                  const uint8_t *packed, int64_t out_dim,
                                  float weight_scale, int threads,
                                  float *scales, int8_t *q, int32_t *acc, float *y)
{
    if (hidden % 4 != 0) return -2;
    for (int64_t r = 0; r < rows; ++r) {
        scales[r] = nslo_absmax_scale_row(x + r * hidden, hidden);
        nslo_quantize_row_int8(x + r * hidden, hidden, scales[r], q + r * hidden);
    }
    bl_ctx c = { x, rows, hidden, packed, out_dim, weight_scale, scales, q, acc, y, 0 };
    nslo_parallel_for(out_dim, threads, bl_cols, &c);
    return c.bad ? -1 : 0;
}

/* ------------------------------------------------------------------------- */
/* Deterministic generators the reference tests use                           */
/* ------------------------------------------------------------------------- */

/* crates/nsl-codegen/tests/bitnet_reference_impl.rs:145-150  lcg_next. */
uint64_t nslo_lcg_next(uint64_t *state)
{
    *state = *state * 6364136223846793005ULL + 1442695040888963407ULL;
    return *state;
}

/* crates/nsl-codegen/tests/bitnet_reference_impl.rs:163-181  make_f10_inputs.
 * acts[128], weights[128*4] ([hidden][out]).  logf/cosf come from the host libm,
 * so activations agree with the committed fixture to ~1 ulp, the trits exactly. */
void nslo_make_f10_inputs(float *acts, int8_t *weights)
{
    uint64_t st = 42;
    for (int i = 0; i < 128; ++i) {
        float u1 = (float)(nslo_lcg_next(&st) >> 32) / (float)UINT32_MAX;
        float u2 = (float)(nslo_lcg_next(&st) >> 32) / (float)UINT32_MAX;
        float m = fmaxf(u1, 1e-9f);
        acts[i] = sqrtf(-2.0f * logf(m)) * cosf(2.0f * 3.14159265358979323846f * u2);
    }
    for (int i = 0; i < 128 * 4; ++i)
        weights[i] = (int8_t)((nslo_lcg_next(&st) >> 32) % 3) - 1;
}

/* crates/nsl-codegen/tests/bitnet_gpu_correctness.rs:587-625  random-case
 * generator: acts uniform in [-1,1) from the top 24 LCG bits, then trits
 * [hidden][out]. */
void nslo_make_gpu_random_case(int64_t rows, int64_t hidden, int64_t out_dim,
                               float *acts, int8_t *weights_kn)
{
    uint64_t st = 0xB175E700D1CEF00DULL ^ ((uint64_t)hidden << 17) ^ (uint64_t)out_dim;
    for (int64_t i = 0; i < rows * hidden; ++i)
        acts[i] = (float)(nslo_lcg_next(&st) >> 40) / 8388608.0f - 1.0f;
    for (int64_t i = 0; i < hidden * out_dim; ++i)
        weights_kn[i] = (int8_t)((nslo_lcg_next(&st) >> 32) % 3) - 1;
}

/* ------------------------------------------------------------------------- */
/* QuantizedTensor (INT8 / INT4 RTN, asymmetric affine)                       */
/* ------------------------------------------------------------------------- */

/* crates/nsl-runtime/src/quantize.rs:187-216  int4_pack / int4_unpack:
 * two codes per byte over the flat row-major index, low nibble = even index. */
static inline void int4_pack(uint8_t *d, int64_t idx, uint8_t v)
{
    if ((idx & 1) == 0) d[idx / 2] |= (uint8_t)(v & 0x0F);
    else d[idx / 2] |= (uint8_t)((v & 0x0F) << 4);
}
static inline uint8_t int4_unpack(const uint8_t *d, int64_t idx)
{
    uint8_t b = d[idx / 2];
    return (idx & 1) == 0 ? (uint8_t)(b & 0x0F) : (uint8_t)((b >> 4) & 0x0F);
}
uint8_t nslo_int4_unpack(const uint8_t *d, int64_t idx) { return int4_unpack(d, idx); }

/* Rust `f64 as u8`: saturating, NaN -> 0. */
static inline uint8_t sat_u8(double v)
{
    if (v != v) return 0;
    if (v <= 0.0) return 0;
    if (v >= 255.0) return 255;
    return (uint8_t)v;
}
static inline double clampd(double v, double lo, double hi)
{
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

/* crates/nsl-runtime/src/quantize.rs:224-254  compute_scale_zp. */
void nslo_compute_scale_zp(const double *v, int64_t n, double qmin, double qmax,
                           float *scale_out, uint8_t *zp_out)
{
    if (n == 0) { *scale_out = 1.0f; *zp_out = 0; return; }
    double mn = INFINITY, mx = -INFINITY;
    for (int64_t i = 0; i < n; ++i) {
        if (v[i] < mn) mn = v[i];
        if (v[i] > mx) mx = v[i];
    }
    double range = mx - mn;
    if (range < 1e-7) {
        double mid_q = round((qmin + qmax) / 2.0);
        double abs_val = fmax(fabs(mn), 1e-7);
        double scale = abs_val / mid_q;
        *zp_out = sat_u8(clampd(round(mid_q - mn / scale), qmin, qmax));
        *scale_out = (float)scale;
        return;
    }
    double scale = range / (qmax - qmin);
    *zp_out = sat_u8(clampd(round(-mn / scale), qmin, qmax));
    *scale_out = (float)scale;
}

/* crates/nsl-runtime/src/quantize.rs:257-260  quantize_val. */
static inline uint8_t quantize_val(double x, float scale, uint8_t zp, double qmin, double qmax)
{
    return sat_u8(clampd(round(x / (double)scale + (double)zp), qmin, qmax));
}
/* crates/nsl-runtime/src/quantize.rs:263-266  dequantize_val. */
static inline double dequantize_val(uint8_t q, float scale, uint8_t zp)
{
    return ((double)q - (double)zp) * (double)scale;
}
double nslo_dequantize_val(uint8_t q, float scale, uint8_t zp) { return dequantize_val(q, scale, zp); }

/* crates/nsl-runtime/src/quantize.rs:72-96  compute_num_scales. */
int64_t nslo_qtensor_num_scales(const int64_t *shape, int64_t ndim, int64_t gran,
                                int64_t axis, int64_t gs)
{
    if (gran == 0) return 1;
    if (ndim == 0) return 1;
    if (gran == 1) return shape[axis];
    if (gran == 2) {
        int64_t ng = (shape[axis] + gs - 1) / gs, outer = 1;
        for (int64_t i = 0; i < ndim; ++i) if (i != axis) outer *= shape[i];
        return outer * ng;
    }
    return 1;
}

static void axis_sizes(const int64_t *shape, int64_t ndim, int64_t axis, int64_t total,
                       int64_t *axis_size, int64_t *inner, int64_t *outer)
{
    *axis_size = shape[axis];
    *inner = 1;
    for (int64_t d = axis + 1; d < ndim; ++d) *inner *= shape[d];
    *outer = total / (*axis_size * *inner);
}

/* crates/nsl-runtime/src/quantize.rs:283-426  nsl_qtensor_quantize.
 * dtype 0 = INT8, 1 = INT4; gran 0/1/2 = tensor/channel/group.  `data` must be
 * zeroed by the caller for INT4 (the reference uses a zeroed allocation).
 * Returns -1 on an unknown dtype/granularity (the reference aborts). */
int nslo_qtensor_quantize(const double *src, const int64_t *shape, int64_t ndim,
                          int64_t dtype, int64_t gran, int64_t axis, int64_t gs,
                          uint8_t *data, float *scale, uint8_t *zp)
{
    if (dtype != 0 && dtype != 1) return -1;
    const double qmin = 0.0, qmax = dtype == 1 ? 15.0 : 255.0;
    int64_t total = 1;
    for (int64_t i = 0; i < ndim; ++i) total *= shape[i];

    if (gran == 0) {
        nslo_compute_scale_zp(src, total, qmin, qmax, &scale[0], &zp[0]);
        for (int64_t i = 0; i < total; ++i) {
            uint8_t qv = quantize_val(src[i], scale[0], zp[0], qmin, qmax);
            if (dtype == 1) int4_pack(data, i, qv); else data[i] = qv;
        }
        return 0;
    }
    int64_t axis_size, inner, outer;
    axis_sizes(shape, ndim, axis, total, &axis_size, &inner, &outer);
    if (gran == 1) {
        double *vals = (double *)malloc(sizeof(double) * (size_t)(outer * inner));
        for (int64_t ch = 0; ch < axis_size; ++ch) {
            int64_t n = 0;
            for (int64_t o = 0; o < outer; ++o)
                for (int64_t in = 0; in < inner; ++in)
                    vals[n++] = src[o * axis_size * inner + ch * inner + in];
            nslo_compute_scale_zp(vals, n, qmin, qmax, &scale[ch], &zp[ch]);
            int64_t vi = 0;
            for (int64_t o = 0; o < outer; ++o)
                for (int64_t in = 0; in < inner; ++in) {
                    int64_t idx = o * axis_size * inner + ch * inner + in;
                    uint8_t qv = quantize_val(vals[vi++], scale[ch], zp[ch], qmin, qmax);
                    if (dtype == 1) int4_pack(data, idx, qv); else data[idx] = qv;
                }
        }
        free(vals);
        return 0;
    }
    if (gran == 2) {
        int64_t ng = (axis_size + gs - 1) / gs, sidx = 0;
        double *vals = (double *)malloc(sizeof(double) * (size_t)(gs * inner));
        for (int64_t o = 0; o < outer; ++o)
            for (int64_t g = 0; g < ng; ++g) {
                int64_t start = g * gs, end = start + gs < axis_size ? start + gs : axis_size;
                int64_t n = 0;
                for (int64_t ch = start; ch < end; ++ch)
                    for (int64_t in = 0; in < inner; ++in)
                        vals[n++] = src[o * axis_size * inner + ch * inner + in];
                nslo_compute_scale_zp(vals, n, qmin, qmax, &scale[sidx], &zp[sidx]);
                int64_t vi = 0;
                for (int64_t ch = start; ch < end; ++ch)
                    for (int64_t in = 0; in < inner; ++in) {
                        int64_t idx = o * axis_size * inner + ch * inner + in;
                        uint8_t qv = quantize_val(vals[vi++], scale[sidx], zp[sidx], qmin, qmax);
                        if (dtype == 1) int4_pack(data, idx, qv); else data[idx] = qv;
                    }
                ++sidx;
            }
        free(vals);
        return 0;
    }
    return -1;
}

/* crates/nsl-runtime/src/quantize.rs:436-537  nsl_qtensor_dequantize (f64 out). */
int nslo_qtensor_dequantize(const uint8_t *data, const float *scale, const uint8_t *zp,
                            const int64_t *shape, int64_t ndim, int64_t dtype,
                            int64_t gran, int64_t axis, int64_t gs, double *out)
{
    if (dtype != 0 && dtype != 1) return -1;
    int64_t total = 1;
    for (int64_t i = 0; i < ndim; ++i) total *= shape[i];
#define QAT(i) (dtype == 1 ? int4_unpack(data, (i)) : data[(i)])
    if (gran == 0) {
        for (int64_t i = 0; i < total; ++i) out[i] = dequantize_val(QAT(i), scale[0], zp[0]);
        return 0;
    }
    int64_t axis_size, inner, outer;
    axis_sizes(shape, ndim, axis, total, &axis_size, &inner, &outer);
    if (gran == 1) {
        for (int64_t o = 0; o < outer; ++o)
            for (int64_t ch = 0; ch < axis_size; ++ch)
                for (int64_t in = 0; in < inner; ++in) {
                    int64_t idx = o * axis_size * inner + ch * inner + in;
                    out[idx] = dequantize_val(QAT(idx), scale[ch], zp[ch]);
                }
        return 0;
    }
    if (gran == 2) {
        int64_t ng = (axis_size + gs - 1) / gs, sidx = 0;
        for (int64_t o = 0; o < outer; ++o)
            for (int64_t g = 0; g < ng; ++g) {
                int64_t start = g * gs, end = start + gs < axis_size ? start + gs : axis_size;
                for (int64_t ch = start; ch < end; ++ch)
                    for (int64_t in = 0; in < inner; ++in) {
                        int64_t idx = o * axis_size * inner + ch * inner + in;
                        out[idx] = dequantize_val(QAT(idx), scale[sidx], zp[sidx]);
                    }
                ++sidx;
            }
        return 0;
    }
#undef QAT
    return -1;
}

/* crates/nsl-runtime/src/cpu.rs:782-815  tiled_matmul_f64: C[m,n] += A[m,k] B[k,n],
 * 64^3 tiles, tile order jj -> kk -> ii, inner i -> k -> j.  C must be zeroed. */
void nslo_tiled_matmul_f64(const double *a, const double *b, double *c,
                           int64_t m, int64_t k, int64_t n)
{
    const int64_t T = 64;
    for (int64_t jj = 0; jj < n; jj += T) {
        int64_t je = jj + T < n ? jj + T : n;
        for (int64_t kk = 0; kk < k; kk += T) {
            int64_t ke = kk + T < k ? kk + T : k;
            for (int64_t ii = 0; ii < m; ii += T) {
                int64_t ie = ii + T < m ? ii + T : m;
                for (int64_t i = ii; i < ie; ++i)
                    for (int64_t ki = kk; ki < ke; ++ki) {
                        double av = a[i * k + ki];
                        for (int64_t j = jj; j < je; ++j)
                            c[i * n + j] += av * b[ki * n + j];
                    }
            }
        }
    }
}

/* crates/nsl-runtime/src/quantize.rs:547-585  nsl_qtensor_matmul_mixed on CPU:
 * x[m,K] (f64) @ dequantize(qw[K,N]) -> f64 [m,N].  Returns -3 where the
 * reference aborts (qw not 2-D is the caller's check; here: K mismatch). */
int nslo_qtensor_matmul_mixed(const double *x, int64_t m, int64_t x_last,
                              const uint8_t *data, const float *scale, const uint8_t *zp,
                              const int64_t *shape2, int64_t dtype, int64_t gran,
                              int64_t axis, int64_t gs, double *out)
{
    if (x_last != shape2[0]) return -3;
    int64_t K = shape2[0], N = shape2[1];
    double *deq = (double *)malloc(sizeof(double) * (size_t)(K * N));
    int rc = nslo_qtensor_dequantize(data, scale, zp, shape2, 2, dtype, gran, axis, gs, deq);
    if (rc == 0) {
        memset(out, 0, sizeof(double) * (size_t)(m * N));
        nslo_tiled_matmul_f64(x, deq, out, m, K, N);
    }
    free(deq);
    return rc;
}

/* ------------------------------------------------------------------------- */
/* AWQ 4-bit                                                                  */
/* ------------------------------------------------------------------------- */

/* crates/nsl-runtime/src/awq.rs:53-65  compute_group_params. */
void nslo_awq_group_params(const double *g, int64_t n, double *scale, double *zero)
{
    double mn = INFINITY, mx = -INFINITY;
    for (int64_t i = 0; i < n; ++i) { mn = fmin(mn, g[i]); mx = fmax(mx, g[i]); }
    if (fabs(mx - mn) < 1e-10) { *scale = 1.0; *zero = mn; return; }
    *scale = (mx - mn) / 15.0;
    *zero = mn;
}

/* crates/nsl-runtime/src/awq.rs:68-71  quantize_int4 (`as i32` saturates, NaN -> 0). */
uint8_t nslo_awq_quantize_int4(double value, double scale, double zero)
{
    double r = round((value - zero) / scale);
    int32_t q;
    if (r != r) q = 0;
    else if (r <= -2147483648.0) q = INT32_MIN;
    else if (r >= 2147483647.0) q = INT32_MAX;
    else q = (int32_t)r;
    if (q < 0) q = 0;
    if (q > 15) q = 15;
    return (uint8_t)q;
}

/* crates/nsl-runtime/src/awq.rs:74-76  dequantize_int4. */
double nslo_awq_dequantize_int4(uint8_t q, double scale, double zero)
{
    return (double)q * scale + zero;
}

/* crates/nsl-runtime/src/awq.rs:82-98  read_nibble / write_nibble. */
static inline uint8_t read_nibble(const uint8_t *d, int64_t idx)
{
    return (idx & 1) == 0 ? (uint8_t)(d[idx / 2] & 0x0F) : (uint8_t)((d[idx / 2] >> 4) & 0x0F);
}
static inline void write_nibble(uint8_t *d, int64_t idx, uint8_t v)
{
    if ((idx & 1) == 0) d[idx / 2] = (uint8_t)((d[idx / 2] & 0xF0) | (v & 0x0F));
    else d[idx / 2] = (uint8_t)((d[idx / 2] & 0x0F) | ((v & 0x0F) << 4));
}

/* crates/nsl-runtime/src/awq.rs:104-144  awq_quantize_cpu: weights [K,N] f64,
 * data (K*N+1)/2 bytes zeroed by caller, scales/zeros [num_groups*N]. */
void nslo_awq_quantize(const double *w, int64_t k, int64_t n, int64_t gs,
                       uint8_t *data, double *scales, double *zeros)
{
    int64_t ng = (k + gs - 1) / gs;
    double *grp = (double *)malloc(sizeof(double) * (size_t)gs);
    for (int64_t col = 0; col < n; ++col)
        for (int64_t g = 0; g < ng; ++g) {
            int64_t start = g * gs, end = start + gs < k ? start + gs : k;
            for (int64_t r = start; r < end; ++r) grp[r - start] = w[r * n + col];
            double s, z;
            nslo_awq_group_params(grp, end - start, &s, &z);
            scales[g * n + col] = s;
            zeros[g * n + col] = z;
            for (int64_t r = start; r < end; ++r)
                write_nibble(data, r * n + col, nslo_awq_quantize_int4(w[r * n + col], s, z));
        }
    free(grp);
}

/* crates/nsl-runtime/src/awq.rs:147-165  awq_dequantize_cpu. */
void nslo_awq_dequantize(const uint8_t *data, const double *scales, const double *zeros,
                         int64_t k, int64_t n, int64_t gs, double *out)
{
    for (int64_t col = 0; col < n; ++col)
        for (int64_t r = 0; r < k; ++r) {
            int64_t g = r / gs;
            out[r * n + col] = nslo_awq_dequantize_int4(read_nibble(data, r * n + col),
                                                        scales[g * n + col], zeros[g * n + col]);
        }
}

/* crates/nsl-runtime/src/awq.rs:202-226  awq_matmul_cpu: input [M,K] f64,
 * dequantise on the fly, f64 accumulate in ascending k.  threads > 1 splits the
 * (i,j) outputs over POSIX threads (our parallelisation; each output's sum order is
 * unchanged, so the result is identical). */
typedef struct {
    const double *input; int64_t m; const uint8_t *data; const double *scales, *zeros;
    int64_t k, n, gs; double *out;
} awq_ctx;

static void awq_outputs(int64_t b, int64_t e, void *p)
{
    awq_ctx *s = (awq_ctx *)p;
    for (int64_t o = b; o < e; ++o) {
        int64_t i = o / s->n, j = o % s->n;
        double acc = 0.0;
        for (int64_t pk = 0; pk < s->k; ++pk) {
            int64_t g = pk / s->gs;
            double wv = nslo_awq_dequantize_int4(read_nibble(s->data, pk * s->n + j),
                                                 s->scales[g * s->n + j], s->zeros[g * s->n + j]);
            acc += s->input[i * s->k + pk] * wv;
        }
        s->out[o] = acc;
    }
}

void nslo_awq_matmul(const double *input, int64_t m, const uint8_t *data,
                     const double *scales, const double *zeros,
                     int64_t k, int64_t n, int64_t gs, int threads, double *out)
{
    awq_ctx c = { input, m, data, scales, zeros, k, n, gs, out };
    nslo_parallel_for(m * n, threads, awq_outputs, &c);
}

/* crates/nsl-runtime/src/awq.rs:330-383  nsl_awq_pre_scale_weight: f32 weight
 * [k,n] times scales[col]^alpha, all in f32 (powf). */
void nslo_awq_pre_scale_weight(const float *w, int64_t k, int64_t n,
                               const float *scales, float alpha, float *out)
{
    for (int64_t r = 0; r < k; ++r)
        for (int64_t c = 0; c < n; ++c)
            out[r * n + c] = w[r * n + c] * powf(scales[c], alpha);
}

/* ------------------------------------------------------------------------- */
/* W4A16 in the benchmark's storage form                                      */
/* ------------------------------------------------------------------------- */

/* The group-quantised weight of the W4A16 workload, stored the way a
 * QuantizedTensor of shape [N,K], INT4, per-group along axis 1 stores it
 * (crates/nsl-runtime/src/quantize.rs:366-417: scale index n*G + g, codes two
 * per byte over the flat index n*K + k, low nibble = even k), dequantised with
 * `(q - zp) * scale` (quantize.rs:263-266) and multiplied as x @ W^T with an
 * f64 accumulator in ascending k, the order awq_matmul_cpu and
 * tiled_matmul_f64 both use.  x is given in f32 (exact widening of bf16).
 * scale is f32 (exact widening of a bf16 scale).  out is f64 [M,N]. */
typedef struct {
    const float *x; int64_t m; const uint8_t *codes; const float *scale; const uint8_t *zp;
    int64_t n, k, gs; double *out;
} w4_ctx;

static void w4_cols(int64_t j0, int64_t j1, void *p)
{
    w4_ctx *s = (w4_ctx *)p;
    const int64_t k = s->k, gs = s->gs, G = (k + gs - 1) / gs;
    double *wrow = (double *)malloc(sizeof(double) * (size_t)k);
    for (int64_t j = j0; j < j1; ++j) {
        for (int64_t pk = 0; pk < k; ++pk)
            wrow[pk] = dequantize_val(int4_unpack(s->codes, j * k + pk),
                                      s->scale[j * G + pk / gs], s->zp[j * G + pk / gs]);
        for (int64_t i = 0; i < s->m; ++i) {
            double acc = 0.0;
            for (int64_t pk = 0; pk < k; ++pk) acc += (double)s->x[i * k + pk] * wrow[pk];
            s->out[i * s->n + j] = acc;
        }
    }
    free(wrow);
}

void nslo_w4a16_matmul_nk(const float *x, int64_t m, const uint8_t *codes,
                          const float *scale, const uint8_t *zp,
                          int64_t n, int64_t k, int64_t gs, int threads, double *out)
{
    w4_ctx c = { x, m, codes, scale, zp, n, k, gs, out };
    nslo_parallel_for(n, threads, w4_cols, &c);
}

/* Online host cores (what the benchmark reports as `cores`). */
int nslo_max_threads(void)
{
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}
