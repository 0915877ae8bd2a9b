/*
 * CPU oracle for the TurboQuant KV-cache hot paths.  TEST INFRASTRUCTURE ONLY:
 * the shipped library never links, loads or calls anything in this file; only the
 * test-suite, the smoke check and the benchmark's CPU-baseline leg do, as the checker.
 *
 * It restates, in plain C with a fully specified fp32 evaluation order, what the
 * reference computes with PyTorch on the CPU:
 *   - codebook / boundaries            turboquant/codebook.py:16-62, 72-98
 *   - normalized FWHT + seeded signs   turboquant/hadamard.py:21-42, 63-78
 *   - TurboQuantMSE.quantize           turboquant/quantizer.py:77-91 (norm, divide, rotate, bucketize)
 *   - _pack_bits (low-first)           turboquant/quantizer.py:17-39
 *   - cache nibble order (high = even) turboquant/tile.py:37-41
 *   - paged scatter of codes + norm    csrc/include/turboquant/quantize_write_kernel.cuh:409-430,
 *                                      csrc/src/quantize_write_binding.cu:207-269
 *   - dequant-attention path           vllm_backend_fused.py:137-149 (repo root prototype),
 *                                      tests/test_fused_integration.py:127-159
 *   - split-KV merge                   csrc/include/flashinfer_decode_turboquant_combine.cuh:42-77
 *
 * Parity pin: the committed fixtures under tests/golden/ were produced by importing the
 * reference's own Python modules (tests/golden/make_golden.py); tests/test_oracle.py checks
 * every function here against them bit-for-bit (codes, norms) or to 1e-5 (attention).
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math -shared -fPIC  (no FMA contraction: the
 * norm must round the square and the add separately to match torch's CPU reduction).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Lloyd-Max centroids for N(0,1), as tabulated by the reference (codebook.py:16-55).  They
 * are part of the storage format: codes are indices into exactly this table. */
static const double C1[2] = {-0.7978845608028654, 0.7978845608028654};
static const double C2[4] = {-1.5104176088887660, -0.4527800398860679, 0.4527800398860679,
                             1.5104176088887660};
static const double C3[8] = {-2.1519775207392190, -1.3439709227384000, -0.7560052489261838,
                             -0.2451209601065855, 0.2451209601065855,  0.7560052489261838,
                             1.3439709227384000,  2.1519775207392190};
static const double C4[16] = {-2.7326368237440100, -2.0693470280837980, -1.6180344937899930,
                              -1.2562490887894980, -0.9423683558764893, -0.6567591430551046,
                              -0.3880823046410021, -0.1284153814744918, 0.1284153814744918,
                              0.3880823046410021,  0.6567591430551046,  0.9423683558764893,
                              1.2562490887894980,  1.6180344937899930,  2.0693470280837980,
                              2.7326368237440100};

static const double* centroid_table(int bits) {
    switch (bits) {
        case 1: return C1;
        case 2: return C2;
        case 3: return C3;
        default: return C4;
    }
}

/* codebook.py:72-90: python-float (double) products, then rounded to fp32 by torch.tensor. */
void tqo_codebook(int dim, int bits, float* centroids, float* boundaries) {
    const double* c = centroid_table(bits);
    const int n = 1 << bits;
    const double scale = 1.0 / sqrt((double)dim);
    for (int i = 0; i < n; i++) centroids[i] = (float)(c[i] * scale);
    for (int i = 0; i + 1 < n; i++) boundaries[i] = (float)(((c[i] + c[i + 1]) / 2.0) * scale);
}

/* hadamard.py:21-42: butterflies h = 1, 2, ..., d/2 then one multiply by (float)(1/sqrt(d)). */
void tqo_fwht(float* x, int d) {
    for (int h = 1; h < d; h <<= 1) {
        for (int i = 0; i < d; i += 2 * h) {
            for (int k = 0; k < h; k++) {
                float a = x[i + k], b = x[i + k + h];
                x[i + k] = a + b;
                x[i + k + h] = a - b;
            }
        }
    }
    /* torch multiplies the fp32 tensor by a python double scalar: the scalar is first
     * rounded to fp32, then one fp32 multiply. */
    const float s = (float)(1.0 / sqrt((double)d));
    for (int i = 0; i < d; i++) x[i] = x[i] * s;
}

/* hadamard.py:63-69 */
void tqo_rotate(const float* x, const float* signs, int d, int padded, float* y) {
    for (int i = 0; i < padded; i++) y[i] = (i < d ? x[i] : 0.0f) * signs[i];
    tqo_fwht(y, padded);
}

/* hadamard.py:72-78 */
void tqo_inverse_rotate(const float* y, const float* signs, int d, int padded, float* x) {
    float* t = (float*)malloc(sizeof(float) * (size_t)padded);
    memcpy(t, y, sizeof(float) * (size_t)padded);
    tqo_fwht(t, padded);
    for (int i = 0; i < d; i++) x[i] = t[i] * signs[i];
    free(t);
}

/* L2 norm of one contiguous fp32 row exactly as Tensor.norm(dim=-1) evaluates it on the CPU
 * in the torch build the fixtures were made with: eight interleaved accumulators
 * acc[k] += x[8j+k]*x[8j+k] (product rounded, then added: no FMA), combined left to right,
 * then a correctly rounded square root.  A tail shorter than eight is added sequentially to
 * the combined sum.  Pinned by tests/golden for d = 128 (the only size the paged cache uses);
 * d = 64 and 256 are covered by the same fixtures. */
static float row_norm(const float* x, int d) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int full = d & ~7;
    for (int j = 0; j < full; j += 8)
        for (int k = 0; k < 8; k++) {
            float sq = x[j + k] * x[j + k];
            acc[k] = acc[k] + sq;
        }
    float s = acc[0];
    for (int k = 1; k < 8; k++) s = s + acc[k];
    for (int j = full; j < d; j++) {
        float sq = x[j] * x[j];
        s = s + sq;
    }
    return sqrtf(s);
}

/* torch.bucketize(v, boundaries) with right=False: number of boundaries strictly below v.
 * The comparison is written as torch's lower bound writes it, !(b >= v), so that a NaN lands
 * in the last bucket as it does there. */
static int bucketize(float v, const float* b, int nb) {
    int lo = 0, hi = nb;
    while (lo < hi) {
        int mid = lo + ((hi - lo) >> 1);
        if (!(b[mid] >= v)) lo = mid + 1; else hi = mid;
    }
    return lo;
}

/* quantizer.py:77-91 for one vector: indices (padded entries) and the fp32 norm. */
void tqo_quantize_indices(const float* x, int d, int padded, const float* signs, int bits,
                          uint8_t* idx, float* norm_out) {
    float bnd[15], cen[16];
    tqo_codebook(padded, bits, cen, bnd);
    float norm = row_norm(x, d);
    if (!(norm >= 1e-8f)) norm = (norm != norm) ? norm : 1e-8f; /* clamp(min=1e-8); NaN stays */
    float* u = (float*)malloc(sizeof(float) * (size_t)padded);
    float* y = (float*)malloc(sizeof(float) * (size_t)padded);
    for (int i = 0; i < d; i++) u[i] = x[i] / norm;
    tqo_rotate(u, signs, d, padded, y);
    const int nb = (1 << bits) - 1;
    for (int i = 0; i < padded; i++) idx[i] = (uint8_t)bucketize(y[i], bnd, nb);
    *norm_out = norm;
    free(u);
    free(y);
}

/* quantizer.py:17-39: value i of each group of 8/bits sits at bit offset i*bits. */
static void pack_low_first(const uint8_t* idx, int n, int bits, uint8_t* out) {
    const int vpb = 8 / bits;
    const int nbytes = (n + vpb - 1) / vpb;
    for (int b = 0; b < nbytes; b++) {
        unsigned v = 0;
        for (int i = 0; i < vpb; i++) {
            int e = b * vpb + i;
            unsigned code = e < n ? idx[e] : 0;
            v |= code << (i * bits);
        }
        out[b] = (uint8_t)v;
    }
}

/* TurboQuantMSE.quantize over n rows: packed [n, ceil(padded/(8/bits))], norms [n]. */
void tqo_quantize_flat(const float* x, int64_t n, int d, int padded, const float* signs,
                       int bits, uint8_t* packed, float* norms) {
    const int vpb = 8 / bits;
    const int nbytes = (padded + vpb - 1) / vpb;
    uint8_t* idx = (uint8_t*)malloc((size_t)padded);
    for (int64_t r = 0; r < n; r++) {
        tqo_quantize_indices(x + r * d, d, padded, signs, bits, idx, norms + r);
        pack_low_first(idx, padded, bits, packed + r * nbytes);
    }
    free(idx);
}

/* TurboQuantMSE.dequantize (quantizer.py:94-106). */
void tqo_dequantize_flat(const uint8_t* packed, const float* norms, int64_t n, int d, int padded,
                         const float* signs, int bits, float* out) {
    float bnd[15], cen[16];
    tqo_codebook(padded, bits, cen, bnd);
    const int vpb = 8 / bits, mask = (1 << bits) - 1;
    const int nbytes = (padded + vpb - 1) / vpb;
    float* y = (float*)malloc(sizeof(float) * (size_t)padded);
    float* xr = (float*)malloc(sizeof(float) * (size_t)padded);
    for (int64_t r = 0; r < n; r++) {
        for (int e = 0; e < padded; e++) {
            int code = (packed[r * nbytes + e / vpb] >> ((e % vpb) * bits)) & mask;
            y[e] = cen[code];
        }
        tqo_inverse_rotate(y, signs, d, padded, xr);
        for (int e = 0; e < d; e++) out[r * d + e] = xr[e] * norms[r];
    }
    free(y);
    free(xr);
}

/* ---- fp16 helpers (round-to-nearest-even, as torch .to(float16)) ---- */
static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | (ax > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf */
    if (ax < 0x33000001u) return (uint16_t)sign;              /* rounds to zero */
    int e = (int)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7fffffu; }
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    return (uint16_t)(sign | (base + q));
}

static float f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16, e = (h >> 10) & 0x1f, m = h & 0x3ff, x;
    if (e == 0) {
        if (m == 0) x = sign;
        else {
            int s = 0;
            while (!(m & 0x400)) { m <<= 1; s++; }
            x = sign | ((uint32_t)(127 - 15 - s + 1) << 23) | ((m & 0x3ff) << 13);
        }
    } else if (e == 31) x = sign | 0x7f800000u | (m << 13);
    else x = sign | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &x, 4);
    return f;
}

uint16_t tqo_f32_to_f16(float f) { return f32_to_f16(f); }
float tqo_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

/* The production write: quantize K and V rows and scatter them into the paged cache
 * [2][num_blocks][block_size][H][ebs] (quantize_write_binding.cu:207-269 with the torch
 * quantizer's arithmetic and tie rule).  Slot s<0 is skipped.  Bytes 0..qbytes-1 are codes
 * (even dim in the high nibble), then the fp16 norm once per 64-dim chunk; the pad bytes
 * up to ebs are left untouched. */
void tqo_write_kv_cache(uint8_t* kv_cache, int64_t num_blocks, int block_size, int H, int ebs,
                        const float* key, const float* value, int64_t T, int64_t token_stride,
                        const float* signs, const int64_t* slot_mapping, int head_dim) {
    int padded = 1;
    while (padded < head_dim) padded <<= 1;
    const int dc = padded / 64, qbytes = dc * 32;
    const size_t slab = (size_t)num_blocks * block_size * H * ebs;
    uint8_t* idx = (uint8_t*)malloc((size_t)padded);
    for (int kv = 0; kv < 2; kv++) {
        const float* src = kv ? value : key;
        for (int64_t t = 0; t < T; t++) {
            int64_t slot = slot_mapping[t];
            if (slot < 0) continue;
            int64_t block = slot / block_size, entry = slot % block_size;
            for (int h = 0; h < H; h++) {
                float norm;
                tqo_quantize_indices(src + t * token_stride + (int64_t)h * head_dim, head_dim,
                                     padded, signs, 4, idx, &norm);
                uint8_t* dst = kv_cache + kv * slab +
                               ((size_t)block * block_size + entry) * H * ebs + (size_t)h * ebs;
                for (int b = 0; b < qbytes; b++)
                    dst[b] = (uint8_t)((idx[2 * b] << 4) | (idx[2 * b + 1] & 0x0f));
                uint16_t nh = f32_to_f16(norm);
                for (int c = 0; c < dc; c++) memcpy(dst + qbytes + 2 * c, &nh, 2);
            }
        }
    }
    free(idx);
}

/* Dequantize one cache slot to the un-rotated fp32 vector: centroid lookup, inverse
 * rotation, times the stored fp16 norm (vllm_backend_fused.py:137-149 at the repo root). */
static void dequant_slot(const uint8_t* slot, int head_dim, int padded, const float* signs,
                         const float* cen, float* out) {
    float y[256], x[256];
    const int qbytes = padded / 2;
    for (int b = 0; b < qbytes; b++) {
        y[2 * b] = cen[slot[b] >> 4];
        y[2 * b + 1] = cen[slot[b] & 0x0f];
    }
    tqo_inverse_rotate(y, signs, head_dim, padded, x);
    uint16_t nh;
    memcpy(&nh, slot + qbytes, 2);
    float norm = f16_to_f32(nh);
    for (int e = 0; e < head_dim; e++) out[e] = x[e] * norm;
}

void tqo_dequant_cache_rows(const uint8_t* slots, int64_t n, int ebs, int head_dim,
                            const float* signs, float* out) {
    int padded = 1;
    while (padded < head_dim) padded <<= 1;
    float bnd[15], cen[16];
    tqo_codebook(padded, 4, cen, bnd);
    for (int64_t r = 0; r < n; r++)
        dequant_slot(slots + r * ebs, head_dim, padded, signs, cen, out + r * head_dim);
}

/* One decode step over the paged quantized cache: out[b,hq,:] = softmax(q.K^T*scale) V with
 * K^, V^ dequantized as above; accumulation in double.  kv range [kv_begin, kv_end) of each
 * sequence is attended (kv_end<0 means seq_len), which also yields split-KV partials.  lse
 * (optional) is the natural-log log-sum-exp of the scaled scores; an empty range gives
 * out = 0 and lse = -inf.  q is [B, Hq, head_dim] fp32; block_table is [B, max_pages]. */
void tqo_decode_paged(const float* q, int B, int Hq, int H, int head_dim, const uint8_t* kv_cache,
                      int64_t num_blocks, int block_size, int ebs, const int32_t* block_table,
                      int max_pages, const int32_t* seq_lens, const float* signs, float sm_scale,
                      int64_t kv_begin, int64_t kv_end, float* out, float* lse) {
    int padded = 1;
    while (padded < head_dim) padded <<= 1;
    float bnd[15], cen[16];
    tqo_codebook(padded, 4, cen, bnd);
    const size_t slab = (size_t)num_blocks * block_size * H * ebs;
    const int group = Hq / H;
    float* kd = (float*)malloc(sizeof(float) * (size_t)head_dim);
    float* vd = (float*)malloc(sizeof(float) * (size_t)head_dim);
    for (int b = 0; b < B; b++) {
        int64_t len = seq_lens[b];
        int64_t t0 = kv_begin < 0 ? 0 : kv_begin;
        int64_t t1 = (kv_end < 0 || kv_end > len) ? len : kv_end;
        for (int h = 0; h < H; h++) {
            int64_t n = t1 > t0 ? t1 - t0 : 0;
            double* sc = (double*)malloc(sizeof(double) * (size_t)(n > 0 ? n * group : 1));
            float* vall = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n * head_dim : 1));
            for (int64_t t = t0; t < t1; t++) {
                int64_t page = block_table[(int64_t)b * max_pages + t / block_size];
                size_t off = (((size_t)page * block_size + (size_t)(t % block_size)) * H + h) * ebs;
                dequant_slot(kv_cache + off, head_dim, padded, signs, cen, kd);
                dequant_slot(kv_cache + slab + off, head_dim, padded, signs, cen, vd);
                memcpy(vall + (t - t0) * head_dim, vd, sizeof(float) * (size_t)head_dim);
                for (int g = 0; g < group; g++) {
                    const float* qv = q + ((size_t)b * Hq + (size_t)h * group + g) * head_dim;
                    double s = 0;
                    for (int e = 0; e < head_dim; e++) s += (double)qv[e] * (double)kd[e];
                    sc[(t - t0) * group + g] = s * (double)sm_scale;
                }
            }
            for (int g = 0; g < group; g++) {
                size_t row = (size_t)b * Hq + (size_t)h * group + g;
                float* o = out + row * head_dim;
                if (n == 0) {
                    for (int e = 0; e < head_dim; e++) o[e] = 0.f;
                    if (lse) lse[row] = -INFINITY;
                    continue;
                }
                double m = -INFINITY;
                for (int64_t t = 0; t < n; t++) if (sc[t * group + g] > m) m = sc[t * group + g];
                double l = 0;
                double* acc = (double*)calloc((size_t)head_dim, sizeof(double));
                for (int64_t t = 0; t < n; t++) {
                    double p = exp(sc[t * group + g] - m);
                    l += p;
                    const float* vv = vall + t * head_dim;
                    for (int e = 0; e < head_dim; e++) acc[e] += p * (double)vv[e];
                }
                for (int e = 0; e < head_dim; e++) o[e] = (float)(acc[e] / l);
                if (lse) lse[row] = (float)(m + log(l));
                free(acc);
            }
            free(sc);
            free(vall);
        }
    }
    free(kd);
    free(vd);
}

/* Log-sum-exp merge of normalized partial outputs (combine.cuh:42-77 with one consistent
 * log base, natural log here): o = sum_s w_s o_s / sum_s w_s, w_s = exp(lse_s - max).
 * partial_o [S, rows, dim], partial_lse [S, rows]; a split with lse = -inf is empty. */
void tqo_merge_partials(const float* partial_o, const float* partial_lse, int S, int64_t rows,
                        int dim, float* out, float* lse_out) {
    for (int64_t r = 0; r < rows; r++) {
        double m = -INFINITY;
        for (int s = 0; s < S; s++) {
            double v = partial_lse[(int64_t)s * rows + r];
            if (v > m) m = v;
        }
        float* o = out + r * dim;
        if (m == -INFINITY) {
            for (int e = 0; e < dim; e++) o[e] = 0.f;
            if (lse_out) lse_out[r] = -INFINITY;
            continue;
        }
        double wsum = 0;
        for (int s = 0; s < S; s++) wsum += exp((double)partial_lse[(int64_t)s * rows + r] - m);
        for (int e = 0; e < dim; e++) {
            double a = 0;
            for (int s = 0; s < S; s++)
                a += exp((double)partial_lse[(int64_t)s * rows + r] - m) *
                     (double)partial_o[((int64_t)s * rows + r) * dim + e];
            o[e] = (float)(a / wsum);
        }
        if (lse_out) lse_out[r] = (float)(m + log(wsum));
    }
}

/* ---------------------------------------------------------------------------------------------
 * The slot format of vLLM's native backend ("turboquant_4bit_nc") as the reference documents it
 * (docs/reference/vllm-upstream-turboquant-architecture.md:33-94 layout, :100-175 store):
 *   slot = [K codes d/2 | ||k|| fp16 | V codes d/2 | V scale fp16 | V zero fp16], even dim in the
 *   LOW nibble; K: x / (||x|| + 1e-8), Hadamard / sqrt(d) without signs, Lloyd-Max of N(0, 1/d);
 *   V: scale = (max - min) / 15, code = clamp(trunc((v - min) / scale + 1/2), 0, 15), zero = min.
 * PARITY UNPINNED: the reference tree holds no code and no vectors for this format (upstream's
 * kernels live in vLLM); this restates the description.  Choices the description leaves open are
 * made here and in the kernels alike: the norm uses the summation order of row_norm above, the
 * Hadamard product is evaluated as butterflies, a constant V row gets code 0 everywhere.
 * ------------------------------------------------------------------------------------------- */
void tqo_nc_store_rows(const float* k, const float* v, int64_t rows, int d, uint8_t* slots, int slot_bytes) {
    float bnd[15], cen[16];
    tqo_codebook(d, 4, cen, bnd);
    float* y = (float*)malloc(sizeof(float) * (size_t)d);
    uint8_t* idx = (uint8_t*)malloc((size_t)d);
    const int qb = d / 2, kps = qb + 2;
    for (int64_t r = 0; r < rows; r++) {
        const float* kr = k + r * d;
        const float* vr = v + r * d;
        uint8_t* dst = slots + r * slot_bytes;
        const float norm = row_norm(kr, d);
        const float den = norm + 1e-8f;
        for (int i = 0; i < d; i++) y[i] = kr[i] / den;
        tqo_fwht(y, d);
        for (int i = 0; i < d; i++) idx[i] = (uint8_t)bucketize(y[i], bnd, 15);
        for (int b = 0; b < qb; b++) dst[b] = (uint8_t)(idx[2 * b] | (idx[2 * b + 1] << 4));
        const uint16_t nh = f32_to_f16(norm);
        dst[qb] = (uint8_t)(nh & 0xFF);
        dst[qb + 1] = (uint8_t)(nh >> 8);
        float mn = vr[0], mx = vr[0];
        for (int i = 1; i < d; i++) {
            mn = fminf(mn, vr[i]);
            mx = fmaxf(mx, vr[i]);
        }
        const float vs = (mx - mn) / 15.0f;
        for (int i = 0; i < d; i++) {
            float qv = 0.0f;
            if (vs > 0.0f) {
                const float num = vr[i] - mn;
                const float quo = num / vs;
                qv = quo + 0.5f;
            }
            qv = fminf(fmaxf(qv, 0.0f), 15.0f);
            idx[i] = (uint8_t)(int)qv;
        }
        uint8_t* vd = dst + kps;
        for (int b = 0; b < qb; b++) vd[b] = (uint8_t)(idx[2 * b] | (idx[2 * b + 1] << 4));
        const uint16_t sh = f32_to_f16(vs), zh = f32_to_f16(mn);
        vd[qb] = (uint8_t)(sh & 0xFF);
        vd[qb + 1] = (uint8_t)(sh >> 8);
        vd[qb + 2] = (uint8_t)(zh & 0xFF);
        vd[qb + 3] = (uint8_t)(zh >> 8);
    }
    free(y);
    free(idx);
}
