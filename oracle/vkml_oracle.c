/*
 * vkml_oracle.c -- CPU restatement of vkML's CPU backend for the ops the B200
 * backend serves.  TEST INFRASTRUCTURE ONLY: it is the checker the parity tests,
 * the smoke test and bench.py's CPU-baseline leg compare the CUDA path against.
 * Nothing in the product path links, loads or calls it.
 *
 * It takes the same `b200_node` descriptors as the CUDA library, with HOST
 * pointers in `data`, and evaluates them the way vkML's single-threaded CPU
 * backend does: same loop order, same summation tree, same libm calls, no
 * fused multiply-add (build with -ffp-contract=off and without -march flags,
 * as vkML's own CMake build does).
 *
 * Parity of this restatement is pinned two ways (tests/test_oracle.py):
 *   - the known-answer vectors of vkML's own C++ tests (tests/cpp/test_ops.cpp:172-311,
 *     tests/cpp/test_core.cpp:30-62) committed under tests/golden/;
 *   - bit-for-bit comparison with the reference CPU backend itself, compiled
 *     from its own sources into oracle/_ref/ (oracle/Makefile), over randomised
 *     layouts of every op.
 *
 * Each function cites the reference source it follows, as path:line inside the
 * vkML tree.
 */
#include "vkml_b200.h"

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- addressing: src/backend/cpu/iterate.h:33-42 -------------------------- */

static int64_t numel(const b200_tensor* t) {
    int64_t n = 1;
    for (int i = 0; i < t->ndim; ++i) n *= t->dims[i];
    return n;
}

static size_t esize(int dtype) {
    switch (dtype) {
        case B200_F32: return 4;
        case B200_F16: return 2;
        case B200_I32: return 4;
        case B200_I64: return 8;
        case B200_BOOL: return 1;
        default: return 0;
    }
}

/* linear_to_offset: row-major linear index -> byte offset through the strides */
static int64_t lin2off(int64_t linear, const b200_tensor* t) {
    int64_t off = 0;
    for (int i = t->ndim - 1; i >= 0; --i) {
        const int64_t extent = t->dims[i];
        const int64_t idx = linear % extent;
        linear /= extent;
        off += idx * t->strides[i];
    }
    return off;
}

static float ld_f32(const b200_tensor* t, int64_t linear) {
    float v;
    memcpy(&v, (const char*)t->data + lin2off(linear, t), 4);
    return v;
}
static void st_f32(const b200_tensor* t, int64_t linear, float v) {
    memcpy((char*)t->data + lin2off(linear, t), &v, 4);
}
static uint8_t ld_u8(const b200_tensor* t, int64_t linear) {
    return *((const uint8_t*)t->data + lin2off(linear, t));
}
static int64_t ld_i64(const b200_tensor* t, int64_t linear) {
    int64_t v;
    memcpy(&v, (const char*)t->data + lin2off(linear, t), 8);
    return v;
}

/* ---- fp16 conversion: src/core/dtype.cpp:28-70 (round to nearest even) ----- */

static float bits2f(uint32_t w) { float f; memcpy(&f, &w, 4); return f; }
static uint32_t f2bits(float f) { uint32_t w; memcpy(&w, &f, 4); return w; }

static float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    const uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        /* zero or subnormal: man * 2^-24, exact in fp32 */
        const float mag = (float)man * 0x1.0p-24f;
        return bits2f(sign | f2bits(mag));
    }
    if (exp == 31) return bits2f(sign | 0x7F800000u | (man << 13));
    return bits2f(sign | ((exp + 112u) << 23) | (man << 13));
}

static uint16_t float_to_half(float f) {
    const uint32_t w = f2bits(f);
    const uint16_t sign = (uint16_t)((w >> 16) & 0x8000u);
    const uint32_t absw = w & 0x7FFFFFFFu;
    if (absw > 0x7F800000u) return (uint16_t)(sign | 0x7E00u); /* NaN: quiet, empty payload */
    if (absw >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to inf (>= 65520) */
    if (absw < 0x33000001u) return sign;                        /* <= 2^-25 rounds to zero */
    int32_t e = (int32_t)(absw >> 23) - 127;
    uint32_t m = (absw & 0x7FFFFFu) | 0x800000u; /* 24-bit significand */
    int shift;                                    /* bits dropped */
    uint32_t base;
    if (e < -14) { /* subnormal half: value = m * 2^(e-23), unit 2^-24 */
        shift = -e - 1; /* = 13 + (-14 - e) */
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7FFFFFu;
    }
    uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q; /* carry into the exponent is correct */
    return (uint16_t)(sign | (base + q));
}

/* ---- pairwise sum: src/backend/cpu/reduce.h:48-73 --------------------------
 * Midpoint-recursive; a run of <= 32 terms is a plain left-to-right sum. */

typedef float (*load_fn)(const void* ctx, int64_t i);

static float pairwise_sum(load_fn load, const void* ctx, int64_t begin, int64_t end) {
    const int64_t n = end - begin;
    if (n <= 0) return 0.0f;
    if (n <= 32) {
        float acc = 0.0f;
        for (int64_t i = begin; i < end; ++i) acc += load(ctx, i);
        return acc;
    }
    const int64_t mid = begin + n / 2;
    return pairwise_sum(load, ctx, begin, mid) + pairwise_sum(load, ctx, mid, end);
}

/* ---- elementwise: src/backend/cpu/kernels_elementwise.cpp ------------------ */

static float sigmoid_ref(float x) { /* :25-31 */
    if (x >= 0.0f) return 1.0f / (1.0f + expf(-x));
    const float e = expf(x);
    return e / (1.0f + e);
}

static float unary_apply(uint32_t op, float x, const uint8_t* params) {
    switch (op) {
        case B200_OP_NEG: return -x;
        case B200_OP_ABS: return fabsf(x);
        case B200_OP_SIGN: return x > 0.0f ? 1.0f : (x < 0.0f ? -1.0f : 0.0f); /* :75-83 */
        case B200_OP_SQUARE: return x * x;
        case B200_OP_SQRT: return sqrtf(x);
        case B200_OP_RSQRT: return 1.0f / sqrtf(x);
        case B200_OP_RECIPROCAL: return 1.0f / x;
        case B200_OP_EXP: return expf(x);
        case B200_OP_LOG: return logf(x);
        case B200_OP_ERF: return erff(x);
        case B200_OP_ERFC: return erfcf(x);
        case B200_OP_SIN: return sinf(x);
        case B200_OP_COS: return cosf(x);
        case B200_OP_TANH: return tanhf(x);
        case B200_OP_SIGMOID: return sigmoid_ref(x);
        case B200_OP_RELU: return x <= 0.0f ? 0.0f : x; /* :223-231, NaN propagates */
        case B200_OP_GELU: return 0.5f * x * erfcf(-x * 0.70710678118654752440f); /* :33-36 */
        case B200_OP_SILU: return x * sigmoid_ref(x);
        case B200_OP_CLAMP: { /* :292-304 */
            float lo, hi;
            memcpy(&lo, params, 4);
            memcpy(&hi, params + 4, 4);
            const int has_lo = params[8] != 0, has_hi = params[9] != 0;
            if (has_lo && x < lo) return lo;
            if (has_hi && x > hi) return hi;
            return x;
        }
        default: return NAN;
    }
}

static float binary_apply(uint32_t op, float x, float y, const uint8_t* params) {
    switch (op) {
        case B200_OP_ADD: return x + y;
        case B200_OP_SUB: return x - y;
        case B200_OP_MUL: return x * y;
        case B200_OP_DIV: return x / y;
        case B200_OP_POW: return powf(x, y);
        case B200_OP_SCALED_ADD: { /* :256-259: two rounded products, one rounded sum */
            float alpha, beta;
            memcpy(&alpha, params, 4);
            memcpy(&beta, params + 4, 4);
            const float p = x * alpha;
            const float q = y * beta;
            return p + q;
        }
        case B200_OP_MAXIMUM: /* :273-281 */
            if (isnan(x) || isnan(y)) return NAN;
            return x > y ? x : y;
        case B200_OP_MINIMUM:
            if (isnan(x) || isnan(y)) return NAN;
            return x < y ? x : y;
        default: return NAN;
    }
}

static int compare_apply(uint32_t op, float x, float y) {
    switch (op) {
        case B200_OP_EQUAL: return x == y;
        case B200_OP_LESS: return x < y;
        case B200_OP_GREATER: return x > y;
        case B200_OP_LESS_EQUAL: return x <= y;
        case B200_OP_GREATER_EQUAL: return x >= y;
        case B200_OP_NOT_EQUAL: return x != y;
        default: return 0;
    }
}

/* ---- movement: src/backend/cpu/kernels_movement.cpp ------------------------ */

static int k_contiguous(const b200_node* n) { /* :20-40 */
    const int64_t cnt = numel(&n->out);
    const size_t es = esize(n->out.dtype);
    for (int64_t i = 0; i < cnt; ++i) {
        memcpy((char*)n->out.data + lin2off(i, &n->out),
               (const char*)n->src[0].data + lin2off(i, &n->src[0]), es);
    }
    return B200_OK;
}

static int k_cast(const b200_node* n) { /* :52-123 */
    const b200_tensor* a = &n->src[0];
    const b200_tensor* o = &n->out;
    const int from = a->dtype, to = o->dtype;
    if (from == to) return k_contiguous(n);
    const int64_t cnt = numel(o);
    for (int64_t i = 0; i < cnt; ++i) {
        const char* s = (const char*)a->data + lin2off(i, a);
        char* d = (char*)o->data + lin2off(i, o);
        if (from == B200_F32) {
            float v; memcpy(&v, s, 4);
            if (to == B200_I32) { int32_t r = (int32_t)v; memcpy(d, &r, 4); }
            else if (to == B200_I64) { int64_t r = (int64_t)v; memcpy(d, &r, 8); }
            else if (to == B200_BOOL) { *(uint8_t*)d = v != 0.0f ? 1 : 0; }
            else if (to == B200_F16) { uint16_t r = float_to_half(v); memcpy(d, &r, 2); }
            else return B200_DTYPE_ERROR;
        } else if (from == B200_F16 && to == B200_F32) {
            uint16_t h; memcpy(&h, s, 2);
            float r = half_to_float(h); memcpy(d, &r, 4);
        } else if (from == B200_I32) {
            int32_t v; memcpy(&v, s, 4);
            if (to == B200_F32) { float r = (float)v; memcpy(d, &r, 4); }
            else if (to == B200_I64) { int64_t r = (int64_t)v; memcpy(d, &r, 8); }
            else return B200_DTYPE_ERROR;
        } else if (from == B200_I64) {
            int64_t v; memcpy(&v, s, 8);
            if (to == B200_F32) { float r = (float)v; memcpy(d, &r, 4); }
            else if (to == B200_I32) { int32_t r = (int32_t)v; memcpy(d, &r, 4); }
            else return B200_DTYPE_ERROR;
        } else if (from == B200_BOOL) {
            const uint8_t v = *(const uint8_t*)s;
            if (to == B200_F32) { float r = v != 0 ? 1.0f : 0.0f; memcpy(d, &r, 4); }
            else if (to == B200_I64) { int64_t r = v != 0 ? 1 : 0; memcpy(d, &r, 8); }
            else return B200_DTYPE_ERROR;
        } else {
            return B200_DTYPE_ERROR;
        }
    }
    return B200_OK;
}

static int k_full(const b200_node* n) { /* :125-173 */
    double value;
    memcpy(&value, n->params, 8);
    const int64_t cnt = numel(&n->out);
    switch (n->out.dtype) {
        case B200_F32: { const float v = (float)value; for (int64_t i = 0; i < cnt; ++i) ((float*)n->out.data)[i] = v; return B200_OK; }
        case B200_F16: { const uint16_t v = float_to_half((float)value); for (int64_t i = 0; i < cnt; ++i) ((uint16_t*)n->out.data)[i] = v; return B200_OK; }
        case B200_I64: { const int64_t v = (int64_t)value; for (int64_t i = 0; i < cnt; ++i) ((int64_t*)n->out.data)[i] = v; return B200_OK; }
        case B200_I32: { const int32_t v = (int32_t)value; for (int64_t i = 0; i < cnt; ++i) ((int32_t*)n->out.data)[i] = v; return B200_OK; }
        case B200_BOOL: memset(n->out.data, value != 0.0 ? 1 : 0, (size_t)cnt); return B200_OK;
        default: return B200_DTYPE_ERROR;
    }
}

static int k_arange(const b200_node* n) { /* :175-197: double arithmetic, then narrow */
    double start, step;
    memcpy(&start, n->params, 8);
    memcpy(&step, n->params + 8, 8);
    const int64_t cnt = numel(&n->out);
    if (n->out.dtype == B200_F32) {
        for (int64_t i = 0; i < cnt; ++i) ((float*)n->out.data)[i] = (float)(start + (double)i * step);
        return B200_OK;
    }
    if (n->out.dtype == B200_I64) {
        for (int64_t i = 0; i < cnt; ++i) ((int64_t*)n->out.data)[i] = (int64_t)(start + (double)i * step);
        return B200_OK;
    }
    return B200_DTYPE_ERROR;
}

/* Philox4x32-10: src/backend/cpu/philox.h:47-89 */
static float philox_uniform(uint64_t seed, uint64_t offset, uint64_t index) {
    uint32_t c0 = (uint32_t)index, c1 = (uint32_t)(index >> 32);
    uint32_t c2 = (uint32_t)offset, c3 = (uint32_t)(offset >> 32);
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t hi0 = (uint32_t)(p0 >> 32), lo0 = (uint32_t)p0;
        const uint32_t hi1 = (uint32_t)(p1 >> 32), lo1 = (uint32_t)p1;
        c0 = hi1 ^ c1 ^ k0;
        c1 = lo1;
        c2 = hi0 ^ c3 ^ k1;
        c3 = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

static int k_rand(const b200_node* n) { /* :199-209 */
    if (n->out.dtype != B200_F32) return B200_DTYPE_ERROR;
    uint64_t seed, offset;
    memcpy(&seed, n->params, 8);
    memcpy(&offset, n->params + 8, 8);
    const int64_t cnt = numel(&n->out);
    for (int64_t i = 0; i < cnt; ++i) st_f32(&n->out, i, philox_uniform(seed, offset, (uint64_t)i));
    return B200_OK;
}

static int k_slice_backward(const b200_node* n) { /* :226-262 */
    const b200_tensor* g = &n->src[0];
    const b200_tensor* o = &n->out;
    int32_t axis; int64_t start, step;
    memcpy(&axis, n->params, 4);
    memcpy(&start, n->params + 8, 8);
    memcpy(&step, n->params + 24, 8);
    const size_t es = esize(o->dtype);
    memset(o->data, 0, (size_t)numel(o) * es);
    const int64_t cnt = numel(g);
    for (int64_t i = 0; i < cnt; ++i) {
        int64_t idx[B200_MAX_DIMS] = {0, 0, 0, 0};
        int64_t lin = i;
        for (int d = g->ndim - 1; d >= 0; --d) { idx[d] = lin % g->dims[d]; lin /= g->dims[d]; }
        int64_t off = 0;
        for (int d = 0; d < o->ndim; ++d) {
            const int64_t j = d == axis ? start + idx[d] * step : idx[d];
            off += j * o->strides[d];
        }
        memcpy((char*)o->data + off, (const char*)g->data + lin2off(i, g), es);
    }
    return B200_OK;
}

static int k_cat(const b200_node* n) { /* :272-317 */
    const b200_tensor *a = &n->src[0], *b = &n->src[1], *o = &n->out;
    int32_t axis;
    memcpy(&axis, n->params, 4);
    const int64_t cnt = numel(o);
    int64_t inner = 1;
    for (int i = axis + 1; i < o->ndim; ++i) inner *= o->dims[i];
    const int64_t oe = o->dims[axis], ae = a->dims[axis], be = b->dims[axis];
    const size_t es = esize(o->dtype);
    for (int64_t i = 0; i < cnt; ++i) {
        const int64_t rest = i % inner, along = (i / inner) % oe, outer = i / (inner * oe);
        const int from_a = along < ae;
        const int64_t extent = from_a ? ae : be;
        const int64_t pos = from_a ? along : along - ae;
        const int64_t lin = (outer * extent + pos) * inner + rest;
        const b200_tensor* s = from_a ? a : b;
        memcpy((char*)o->data + lin2off(i, o), (const char*)s->data + lin2off(lin, s), es);
    }
    return B200_OK;
}

static int k_index_select(const b200_node* n) { /* :339-369 */
    const b200_tensor *a = &n->src[0], *idx = &n->src[1], *o = &n->out;
    int32_t axis;
    memcpy(&axis, n->params, 4);
    const int64_t cnt = numel(o);
    int64_t inner = 1;
    for (int i = axis + 1; i < o->ndim; ++i) inner *= o->dims[i];
    const int64_t extent = o->dims[axis], ae = a->dims[axis];
    const size_t es = esize(o->dtype);
    for (int64_t i = 0; i < cnt; ++i) {
        const int64_t rest = i % inner, k = (i / inner) % extent, outer = i / (inner * extent);
        const int64_t j = ld_i64(idx, k);
        if (j < 0 || j >= ae) return B200_INDEX_ERROR;
        const int64_t from = (outer * ae + j) * inner + rest;
        memcpy((char*)o->data + lin2off(i, o), (const char*)a->data + lin2off(from, a), es);
    }
    return B200_OK;
}

static int k_scatter_add(const b200_node* n) { /* :381-429: ascending fold into an f32 scratch */
    const b200_tensor *src = &n->src[0], *idx = &n->src[1], *o = &n->out;
    int32_t axis;
    memcpy(&axis, n->params, 4);
    if (o->dtype != B200_F32) return B200_DTYPE_ERROR;
    const int64_t on = numel(o);
    memset(o->data, 0, (size_t)on * 4);
    const int64_t cnt = numel(src);
    if (cnt == 0) return B200_OK;
    int64_t inner = 1;
    for (int i = axis + 1; i < src->ndim; ++i) inner *= src->dims[i];
    const int64_t se = src->dims[axis], oe = o->dims[axis];
    float* acc = (float*)calloc((size_t)(on > 0 ? on : 1), sizeof(float));
    if (!acc) return B200_OUT_OF_MEMORY;
    for (int64_t i = 0; i < cnt; ++i) {
        const int64_t rest = i % inner, k = (i / inner) % se, outer = i / (inner * se);
        const int64_t j = ld_i64(idx, k);
        if (j < 0 || j >= oe) { free(acc); return B200_INDEX_ERROR; }
        acc[(outer * oe + j) * inner + rest] += ld_f32(src, i);
    }
    for (int64_t i = 0; i < on; ++i) st_f32(o, i, acc[i]);
    free(acc);
    return B200_OK;
}

typedef struct { int64_t out_h, out_w, channels; int32_t p[10]; } win_t;
enum { KH, KW, SH, SW, PH, PW, DH, DW, IH, IW };

static win_t window_of(const uint8_t* params, int64_t channels_times_patch) { /* :438-447 */
    win_t w;
    memcpy(w.p, params, sizeof(w.p));
    w.out_h = (w.p[IH] + 2LL * w.p[PH] - ((int64_t)w.p[DH] * (w.p[KH] - 1) + 1)) / w.p[SH] + 1;
    w.out_w = (w.p[IW] + 2LL * w.p[PW] - ((int64_t)w.p[DW] * (w.p[KW] - 1) + 1)) / w.p[SW] + 1;
    w.channels = channels_times_patch / ((int64_t)w.p[KH] * w.p[KW]);
    return w;
}

static int k_im2col(const b200_node* n) { /* :455-483 */
    const b200_tensor *in = &n->src[0], *o = &n->out;
    const win_t w = window_of(n->params, o->dims[1]);
    const int64_t patch = (int64_t)w.p[KH] * w.p[KW], positions = w.out_h * w.out_w;
    for (int64_t b = 0; b < o->dims[0]; ++b)
        for (int64_t row = 0; row < o->dims[1]; ++row) {
            const int64_t c = row / patch, ki = (row % patch) / w.p[KW], kj = (row % patch) % w.p[KW];
            for (int64_t pos = 0; pos < positions; ++pos) {
                const int64_t oh = pos / w.out_w, ow = pos % w.out_w;
                const int64_t h = oh * w.p[SH] - w.p[PH] + ki * w.p[DH];
                const int64_t x = ow * w.p[SW] - w.p[PW] + kj * w.p[DW];
                const int inside = h >= 0 && h < w.p[IH] && x >= 0 && x < w.p[IW];
                const int64_t s = ((b * w.channels + c) * w.p[IH] + h) * w.p[IW] + x;
                st_f32(o, (b * o->dims[1] + row) * positions + pos, inside ? ld_f32(in, s) : 0.0f);
            }
        }
    return B200_OK;
}

static int k_col2im(const b200_node* n) { /* :501-542: pull, terms added in (ki, kj) order */
    const b200_tensor *cols = &n->src[0], *o = &n->out;
    const win_t w = window_of(n->params, cols->dims[1]);
    const int64_t patch = (int64_t)w.p[KH] * w.p[KW], positions = w.out_h * w.out_w;
    const int64_t total = numel(o);
    for (int64_t i = 0; i < total; ++i) {
        const int64_t x = i % w.p[IW], h = (i / w.p[IW]) % w.p[IH];
        const int64_t c = (i / ((int64_t)w.p[IW] * w.p[IH])) % w.channels;
        const int64_t b = i / ((int64_t)w.p[IW] * w.p[IH] * w.channels);
        float acc = 0.0f;
        for (int64_t ki = 0; ki < w.p[KH]; ++ki) {
            const int64_t top = h + w.p[PH] - ki * w.p[DH];
            if (top < 0 || top % w.p[SH] != 0) continue;
            const int64_t oh = top / w.p[SH];
            if (oh >= w.out_h) continue;
            for (int64_t kj = 0; kj < w.p[KW]; ++kj) {
                const int64_t left = x + w.p[PW] - kj * w.p[DW];
                if (left < 0 || left % w.p[SW] != 0) continue;
                const int64_t ow = left / w.p[SW];
                if (ow >= w.out_w) continue;
                const int64_t row = c * patch + ki * w.p[KW] + kj;
                acc += ld_f32(cols, (b * cols->dims[1] + row) * positions + oh * w.out_w + ow);
            }
        }
        st_f32(o, i, acc);
    }
    return B200_OK;
}

/* first strict maximum of a window: :557-580 */
static int64_t argmax_in_window(const win_t* w, const b200_tensor* in, int64_t base, int64_t oh, int64_t ow) {
    float best = -INFINITY;
    int64_t best_offset = -1;
    for (int64_t ki = 0; ki < w->p[KH]; ++ki) {
        const int64_t h = oh * w->p[SH] - w->p[PH] + ki * w->p[DH];
        if (h < 0 || h >= w->p[IH]) continue;
        for (int64_t kj = 0; kj < w->p[KW]; ++kj) {
            const int64_t x = ow * w->p[SW] - w->p[PW] + kj * w->p[DW];
            if (x < 0 || x >= w->p[IW]) continue;
            const float v = ld_f32(in, base + h * w->p[IW] + x);
            if (v > best) { best = v; best_offset = ki * w->p[KW] + kj; }
        }
    }
    return best_offset;
}

static int k_max_pool2d(const b200_node* n) { /* :585-610 */
    const b200_tensor *in = &n->src[0], *o = &n->out;
    const win_t w = window_of(n->params, 1);
    const int64_t out_h = o->dims[2], out_w = o->dims[3], planes = o->dims[0] * o->dims[1];
    for (int64_t plane = 0; plane < planes; ++plane) {
        const int64_t base = plane * w.p[IH] * w.p[IW];
        for (int64_t oh = 0; oh < out_h; ++oh)
            for (int64_t ow = 0; ow < out_w; ++ow) {
                const int64_t off = argmax_in_window(&w, in, base, oh, ow);
                if (off < 0) return B200_INTERNAL_ERROR;
                const int64_t h = oh * w.p[SH] - w.p[PH] + (off / w.p[KW]) * w.p[DH];
                const int64_t x = ow * w.p[SW] - w.p[PW] + (off % w.p[KW]) * w.p[DW];
                st_f32(o, (plane * out_h + oh) * out_w + ow, ld_f32(in, base + h * w.p[IW] + x));
            }
    }
    return B200_OK;
}

static int k_max_pool2d_backward(const b200_node* n) { /* :629-680 */
    const b200_tensor *grad = &n->src[0], *in = &n->src[1], *o = &n->out;
    const win_t w = window_of(n->params, 1);
    const int64_t out_h = grad->dims[2], out_w = grad->dims[3], planes = o->dims[0] * o->dims[1];
    for (int64_t plane = 0; plane < planes; ++plane) {
        const int64_t base = plane * w.p[IH] * w.p[IW];
        for (int64_t h = 0; h < w.p[IH]; ++h)
            for (int64_t x = 0; x < w.p[IW]; ++x) {
                float acc = 0.0f;
                for (int64_t ki = 0; ki < w.p[KH]; ++ki) {
                    const int64_t top = h + w.p[PH] - ki * w.p[DH];
                    if (top < 0 || top % w.p[SH] != 0) continue;
                    const int64_t oh = top / w.p[SH];
                    if (oh >= out_h) continue;
                    for (int64_t kj = 0; kj < w.p[KW]; ++kj) {
                        const int64_t left = x + w.p[PW] - kj * w.p[DW];
                        if (left < 0 || left % w.p[SW] != 0) continue;
                        const int64_t ow = left / w.p[SW];
                        if (ow >= out_w) continue;
                        if (argmax_in_window(&w, in, base, oh, ow) == ki * w.p[KW] + kj)
                            acc += ld_f32(grad, (plane * out_h + oh) * out_w + ow);
                    }
                }
                st_f32(o, base + h * w.p[IW] + x, acc);
            }
    }
    return B200_OK;
}

static int k_tri(const b200_node* n, int upper) { /* kernels_elementwise.cpp:326-352 */
    const b200_tensor *in = &n->src[0], *o = &n->out;
    int32_t diagonal;
    memcpy(&diagonal, n->params, 4);
    const int nd = o->ndim;
    const int64_t width = o->dims[nd - 1], height = o->dims[nd - 2], cnt = numel(o);
    for (int64_t i = 0; i < cnt; ++i) {
        const int64_t col = i % width, row = (i / width) % height, d = col - row;
        const int keep = upper ? d >= diagonal : d <= diagonal;
        st_f32(o, i, keep ? ld_f32(in, i) : 0.0f);
    }
    return B200_OK;
}

/* ---- reductions: src/backend/cpu/kernels_reduce.cpp, reduce.cpp:11-30 ------ */

typedef struct {
    b200_tensor kept, reduced;
} plan_t;

static plan_t make_plan(const b200_tensor* in, uint32_t mask) {
    plan_t p;
    memset(&p, 0, sizeof(p));
    p.kept.dtype = p.reduced.dtype = in->dtype;
    for (int i = 0; i < in->ndim; ++i) {
        b200_tensor* t = (mask & (1u << i)) ? &p.reduced : &p.kept;
        t->dims[t->ndim] = in->dims[i];
        t->strides[t->ndim] = in->strides[i];
        t->ndim++;
    }
    return p;
}

typedef struct {
    const char* data;
    int64_t base;
    const b200_tensor* reduced;
    float peak;
} reader_t;

static float read_at(const void* ctx, int64_t k) {
    const reader_t* r = (const reader_t*)ctx;
    float v;
    memcpy(&v, r->data + r->base + lin2off(k, r->reduced), 4);
    return v;
}
static float read_exp_shifted(const void* ctx, int64_t k) {
    const reader_t* r = (const reader_t*)ctx;
    return expf(read_at(ctx, k) - r->peak);
}

static int k_reduce(const b200_node* n) {
    const b200_tensor *in = &n->src[0], *o = &n->out;
    uint32_t mask;
    memcpy(&mask, n->params, 4);
    if (mask == 0) mask = in->ndim <= 0 ? 0u : (1u << in->ndim) - 1u;
    const plan_t plan = make_plan(in, mask);
    const int64_t n_out = numel(&plan.kept), n_red = numel(&plan.reduced);
    for (int64_t oi = 0; oi < n_out; ++oi) {
        reader_t r = {(const char*)in->data, lin2off(oi, &plan.kept), &plan.reduced, 0.0f};
        float fv = 0.0f;
        int64_t iv = 0;
        switch (n->op) {
            case B200_OP_SUM: fv = pairwise_sum(read_at, &r, 0, n_red); break; /* :94-96 */
            case B200_OP_MEAN: /* :98-107 */
                fv = n_red == 0 ? NAN : pairwise_sum(read_at, &r, 0, n_red) / (float)n_red;
                break;
            case B200_OP_PROD: { /* :109-118 */
                fv = 1.0f;
                for (int64_t i = 0; i < n_red; ++i) fv *= read_at(&r, i);
                break;
            }
            case B200_OP_MAX: { /* :120-135: the first NaN wins */
                fv = -INFINITY;
                for (int64_t i = 0; i < n_red; ++i) {
                    const float v = read_at(&r, i);
                    if (isnan(v)) { fv = v; break; }
                    if (v > fv) fv = v;
                }
                break;
            }
            case B200_OP_MIN: { /* :137-152 */
                fv = INFINITY;
                for (int64_t i = 0; i < n_red; ++i) {
                    const float v = read_at(&r, i);
                    if (isnan(v)) { fv = v; break; }
                    if (v < fv) fv = v;
                }
                break;
            }
            case B200_OP_ARGMAX: { /* :160-176: strict >, NaN never selected */
                float best = -INFINITY;
                for (int64_t i = 0; i < n_red; ++i) {
                    const float v = read_at(&r, i);
                    if (v > best) { best = v; iv = i; }
                }
                break;
            }
            case B200_OP_ARGMIN: { /* :178-192 */
                float best = INFINITY;
                for (int64_t i = 0; i < n_red; ++i) {
                    const float v = read_at(&r, i);
                    if (v < best) { best = v; iv = i; }
                }
                break;
            }
            default: return B200_NOT_IMPLEMENTED;
        }
        if (n->op == B200_OP_ARGMAX || n->op == B200_OP_ARGMIN) ((int64_t*)o->data)[oi] = iv;
        else ((float*)o->data)[oi] = fv;
    }
    return B200_OK;
}

static int k_softmax(const b200_node* n, int log_form) { /* :206-245 */
    const b200_tensor *in = &n->src[0], *o = &n->out;
    int32_t axis;
    memcpy(&axis, n->params, 4);
    const uint32_t mask = 1u << (uint32_t)axis;
    const plan_t plan = make_plan(in, mask), oplan = make_plan(o, mask);
    const int64_t n_out = numel(&plan.kept), n_axis = numel(&plan.reduced);
    for (int64_t oi = 0; oi < n_out; ++oi) {
        reader_t r = {(const char*)in->data, lin2off(oi, &plan.kept), &plan.reduced, 0.0f};
        const int64_t out_base = lin2off(oi, &oplan.kept);
        float peak = -INFINITY;
        for (int64_t k = 0; k < n_axis; ++k) { /* std::max(peak, v): a NaN v is ignored */
            const float v = read_at(&r, k);
            peak = peak < v ? v : peak;
        }
        r.peak = peak;
        const float denom = pairwise_sum(read_exp_shifted, &r, 0, n_axis);
        for (int64_t k = 0; k < n_axis; ++k) {
            const float shifted = read_at(&r, k) - peak;
            const float v = log_form ? shifted - logf(denom) : expf(shifted) / denom;
            memcpy((char*)o->data + out_base + lin2off(k, &oplan.reduced), &v, 4);
        }
    }
    return B200_OK;
}

/* ---- matmul: src/backend/cpu/kernels_matmul.cpp:35-87 ---------------------- */

typedef struct {
    const char *a, *b;
    int64_t a_k, b_k;
} dot_t;

static float dot_term(const void* ctx, int64_t i) {
    const dot_t* d = (const dot_t*)ctx;
    float x, y;
    memcpy(&x, d->a + i * d->a_k, 4);
    memcpy(&y, d->b + i * d->b_k, 4);
    return x * y; /* product rounded on its own; the sum is the pairwise tree */
}

static int k_matmul(const b200_node* n) {
    const b200_tensor *a = &n->src[0], *b = &n->src[1], *o = &n->out;
    if (o->ndim != 4 || a->ndim != 4 || b->ndim != 4) return B200_SHAPE_ERROR;
    const int64_t b0 = o->dims[0], b1 = o->dims[1], m = o->dims[2], nn = o->dims[3], k = a->dims[3];
    if (b->dims[2] != k) return B200_SHAPE_ERROR;
    float* out = (float*)o->data;
    for (int64_t i0 = 0; i0 < b0; ++i0)
        for (int64_t i1 = 0; i1 < b1; ++i1) {
            const int64_t ab = i0 * a->strides[0] + i1 * a->strides[1];
            const int64_t bb = i0 * b->strides[0] + i1 * b->strides[1];
            const int64_t ob = (i0 * b1 + i1) * m * nn;
            for (int64_t r = 0; r < m; ++r)
                for (int64_t c = 0; c < nn; ++c) {
                    dot_t d = {(const char*)a->data + ab + r * a->strides[2],
                               (const char*)b->data + bb + c * b->strides[3], a->strides[3], b->strides[2]};
                    out[ob + r * nn + c] = pairwise_sum(dot_term, &d, 0, k);
                }
        }
    return B200_OK;
}

/* ---- dispatch: src/backend/cpu/cpu_backend.cpp:60-91 ----------------------- */

static int is_view_or_leaf(uint32_t op) {
    return op == B200_OP_INPUT || op == B200_OP_CONST || (op >= B200_OP_RESHAPE && op <= B200_OP_UNSQUEEZE);
}

static int compute_one(const b200_node* n) {
    const uint32_t op = n->op;
    const int64_t cnt = numel(&n->out);
    if (op >= B200_OP_NEG && op <= B200_OP_CLAMP) {
        if (n->out.dtype != B200_F32) return B200_DTYPE_ERROR;
        for (int64_t i = 0; i < cnt; ++i) st_f32(&n->out, i, unary_apply(op, ld_f32(&n->src[0], i), n->params));
        return B200_OK;
    }
    if ((op >= B200_OP_ADD && op <= B200_OP_MINIMUM)) {
        if (n->out.dtype != B200_F32) return B200_DTYPE_ERROR;
        for (int64_t i = 0; i < cnt; ++i)
            st_f32(&n->out, i, binary_apply(op, ld_f32(&n->src[0], i), ld_f32(&n->src[1], i), n->params));
        return B200_OK;
    }
    if (op >= B200_OP_EQUAL && op <= B200_OP_NOT_EQUAL) {
        if (n->out.dtype != B200_BOOL || n->src[0].dtype != B200_F32) return B200_DTYPE_ERROR;
        for (int64_t i = 0; i < cnt; ++i)
            *((uint8_t*)n->out.data + lin2off(i, &n->out)) =
                compare_apply(op, ld_f32(&n->src[0], i), ld_f32(&n->src[1], i)) ? 1 : 0;
        return B200_OK;
    }
    switch (op) {
        case B200_OP_WHERE: /* kernels_elementwise.cpp:370-397 */
            if (n->out.dtype != B200_F32) return B200_DTYPE_ERROR;
            for (int64_t i = 0; i < cnt; ++i)
                st_f32(&n->out, i, ld_u8(&n->src[0], i) != 0 ? ld_f32(&n->src[1], i) : ld_f32(&n->src[2], i));
            return B200_OK;
        case B200_OP_FULL: return k_full(n);
        case B200_OP_ARANGE: return k_arange(n);
        case B200_OP_RAND: return k_rand(n);
        case B200_OP_CONTIGUOUS: return k_contiguous(n);
        case B200_OP_CAST: return k_cast(n);
        case B200_OP_CAT: return k_cat(n);
        case B200_OP_TRIU: return k_tri(n, 1);
        case B200_OP_TRIL: return k_tri(n, 0);
        case B200_OP_SUM: case B200_OP_MEAN: case B200_OP_MAX: case B200_OP_MIN: case B200_OP_PROD:
        case B200_OP_ARGMAX: case B200_OP_ARGMIN: return k_reduce(n);
        case B200_OP_MATMUL: return k_matmul(n);
        case B200_OP_SOFTMAX: return k_softmax(n, 0);
        case B200_OP_LOG_SOFTMAX: return k_softmax(n, 1);
        case B200_OP_IM2COL: return k_im2col(n);
        case B200_OP_COL2IM: return k_col2im(n);
        case B200_OP_MAX_POOL2D: return k_max_pool2d(n);
        case B200_OP_MAX_POOL2D_BACKWARD: return k_max_pool2d_backward(n);
        case B200_OP_INDEX_SELECT: return k_index_select(n);
        case B200_OP_SCATTER_ADD: return k_scatter_add(n);
        case B200_OP_SLICE_BACKWARD: return k_slice_backward(n);
        default: return B200_NOT_IMPLEMENTED;
    }
}

/* F16 is storage, never arithmetic (kernels_elementwise.cpp:89-99): every kernel of the CPU
 * backend widens Half to float on load, computes in float and narrows once, round-to-nearest-even,
 * on store (reduce_generic<Half, ...> kernels_reduce.cpp:45-92, softmax_impl<Log, Half> :206-251,
 * matmul_impl<Half> kernels_matmul.cpp:35-92, the movement kernels kernels_movement.cpp:685-709).
 * So a node that touches F16 is the same node on widened copies with the result narrowed. */
static void dense_like(const b200_tensor* t, int dtype, void* data, b200_tensor* out) {
    *out = *t;
    out->dtype = dtype;
    out->data = data;
    int64_t stride = (int64_t)esize(dtype);
    for (int d = t->ndim - 1; d >= 0; --d) {
        out->strides[d] = stride;
        stride *= t->dims[d];
    }
}

static int compute_f16(const b200_node* n) {
    b200_node w = *n;
    void* temps[B200_MAX_SRC + 1] = {0};
    int rc = B200_OK;
    for (uint32_t s = 0; s < n->n_src && rc == B200_OK; ++s) {
        if (n->src[s].dtype != B200_F16) continue;
        const int64_t cnt = numel(&n->src[s]);
        temps[s] = malloc((size_t)(cnt > 0 ? cnt : 1) * 4);
        b200_node c;
        memset(&c, 0, sizeof c);
        c.op = B200_OP_CAST;
        c.n_src = 1;
        c.src[0] = n->src[s];
        dense_like(&n->src[s], B200_F32, temps[s], &c.out);
        rc = k_cast(&c);
        w.src[s] = c.out;
    }
    if (rc == B200_OK && n->out.dtype == B200_F16) {
        const int64_t cnt = numel(&n->out);
        temps[B200_MAX_SRC] = malloc((size_t)(cnt > 0 ? cnt : 1) * 4);
        dense_like(&n->out, B200_F32, temps[B200_MAX_SRC], &w.out);
    }
    if (rc == B200_OK) rc = compute_one(&w);
    if (rc == B200_OK && n->out.dtype == B200_F16) {
        b200_node c;
        memset(&c, 0, sizeof c);
        c.op = B200_OP_CAST;
        c.n_src = 1;
        c.src[0] = w.out;
        c.out = n->out;
        rc = k_cast(&c);
    }
    for (int i = 0; i <= B200_MAX_SRC; ++i) free(temps[i]);
    return rc;
}

static int touches_f16(const b200_node* n) {
    if (n->op == B200_OP_CAST || n->op == B200_OP_FULL) return 0; /* handle F16 themselves */
    if (n->out.dtype == B200_F16) return 1;
    for (uint32_t s = 0; s < n->n_src; ++s)
        if (n->src[s].dtype == B200_F16) return 1;
    return 0;
}

/* Evaluate `n_nodes` descriptors in order on host memory. Returns a b200_status. */
int vkml_oracle_compute(const b200_node* nodes, size_t n_nodes) {
    for (size_t i = 0; i < n_nodes; ++i) {
        if (is_view_or_leaf(nodes[i].op)) continue;
        const int rc = touches_f16(&nodes[i]) ? compute_f16(&nodes[i]) : compute_one(&nodes[i]);
        if (rc != B200_OK) return rc;
    }
    return B200_OK;
}

/* Exposed for the fp16 table test (tests/cpp/test_core.cpp:30-62 in vkML). */
uint16_t vkml_oracle_f32_to_f16(float f) { return float_to_half(f); }
float vkml_oracle_f16_to_f32(uint16_t h) { return half_to_float(h); }
float vkml_oracle_philox_uniform(uint64_t seed, uint64_t offset, uint64_t index) { return philox_uniform(seed, offset, index); }
