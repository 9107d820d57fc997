/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the W4A16 quantised-linear path.
 *
 * A plain-C restatement of the reference algorithm (kiln's `kiln-marlin-gemm`
 * crate, paths below are relative to the kiln project root).  Nothing in the
 * product (`kiln_b200/`) may import, link or call this file; only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg use it, and
 * there only as the checker / the timed CPU baseline.
 *
 * What pins this oracle:
 *   - The packed-weight and permuted-scale FORMAT (steps a2/a3) is PARITY UNPINNED in the strict sense: the
 *     reference holds no golden vector, known-answer test or fixture for the packed bytes, its Rust packer cannot be
 *     built here (no cargo/rustc), and its CUDA kernel, compiled unmodified for sm_100a, ended its first launch on a
 *     B200 with "an illegal instruction was encountered" and is not run again.  What holds the format in place is
 *     weaker: this restatement keeps the loop order and temporaries of crates/kiln-marlin-gemm/src/lib.rs:296-357,
 *     429-528; an independent vectorised numpy restatement (oracle/__init__.py) agrees with it bit for bit; and an
 *     unpacker written from the consumer side (`oracle_unpack_fragment`, the mma.m16n8k16 register ownership the
 *     reference kernel feeds, csrc/marlin_kernel.cu:131-152, 442-461) inverts it on every tested shape.
 *   - The QUANTISER (step a1) is pinned against the reference's own numpy
 *     restatement (scripts/c11_marlin_audit.py:208-241) on tie-free inputs;
 *     the tie rule itself (round half away from zero, Rust `f32::round`) has
 *     no golden vector anywhere in the reference: that detail is "parity
 *     unpinned" and follows crates/kiln-marlin-gemm/src/lib.rs:422 by reading.
 *   - The GPTQ layout restated in oracle/__init__.py (`np_gptq_pack`, `np_gptq_dequant`) is pinned to the two
 *     known-answer tests the reference holds for it (crates/kiln-model/src/quantized.rs:311-415), reproduced in
 *     tests/test_oracle_golden.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MAX_Q 15    /* crates/kiln-marlin-gemm/src/lib.rs:288 */
#define Q_OFFSET 8  /* crates/kiln-marlin-gemm/src/lib.rs:289 */

/* ---- scalar format helpers ------------------------------------------------ */

/* f32 -> IEEE binary16 bits, round to nearest even (what `half::f16::from_f32`
 * does; crates/kiln-marlin-gemm/src/lib.rs:411, 488). */
static uint16_t f32_to_f16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t mant = x & 0x007fffffu;
    int32_t exp = (int32_t)((x >> 23) & 0xff);
    if (exp == 0xff) return (uint16_t)(sign | 0x7c00u | (mant ? 0x200u : 0));
    int32_t e = exp - 127 + 15;
    if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        mant |= 0x00800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t half_m = mant >> shift;
        uint32_t rem = mant & ((1u << shift) - 1);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_m & 1))) half_m++;
        return (uint16_t)(sign | half_m);
    }
    uint32_t half_m = mant >> 13;
    uint32_t rem = mant & 0x1fffu;
    uint32_t out = sign | ((uint32_t)e << 10) | half_m;
    if (rem > 0x1000u || (rem == 0x1000u && (half_m & 1))) out++;
    return (uint16_t)out;
}

static float f16_bits_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t mant = h & 0x3ffu;
    uint32_t x;
    if (exp == 0) {
        if (mant == 0) {
            x = sign;
        } else {
            int e = -1;
            do { mant <<= 1; e++; } while (!(mant & 0x400u));
            mant &= 0x3ffu;
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | (mant << 13);
        }
    } else if (exp == 0x1f) {
        x = sign | 0x7f800000u | (mant << 13);
    } else {
        x = sign | ((exp - 15 + 127) << 23) | (mant << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

static float bf16_bits_to_f32(uint16_t b) {
    uint32_t x = (uint32_t)b << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}

/* f32 -> bf16 bits, round to nearest even (candle `to_dtype(BF16)`,
 * crates/kiln-marlin-gemm/tests/parity.rs:96-99). */
static uint16_t f32_to_bf16_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7fffu + lsb;
    return (uint16_t)(x >> 16);
}

uint16_t oracle_f32_to_f16_bits(float f) { return f32_to_f16_bits(f); }
float oracle_f16_bits_to_f32(uint16_t h) { return f16_bits_to_f32(h); }
uint16_t oracle_f32_to_bf16_bits(float f) { return f32_to_bf16_bits(f); }

/* ---- permutation tables ---------------------------------------------------- */

/* crates/kiln-marlin-gemm/src/lib.rs:296-327 (build_weight_perm). */
void oracle_build_weight_perm(int32_t *out /* [1024] */) {
    int32_t perm[1024];
    int p = 0;
    for (int i = 0; i < 32; i++) {
        int32_t perm1[8];
        int c = 0;
        int col = i / 4;
        for (int block = 0; block < 2; block++) {
            int rows[4] = {2 * (i % 4), 2 * (i % 4) + 1, 2 * (i % 4 + 4), 2 * (i % 4 + 4) + 1};
            for (int r = 0; r < 4; r++) perm1[c++] = 16 * rows[r] + col + 8 * block;
        }
        for (int j = 0; j < 4; j++)
            for (int t = 0; t < 8; t++) perm[p++] = perm1[t] + 256 * j;
    }
    static const int inter[8] = {0, 2, 4, 6, 1, 3, 5, 7};
    for (int base = 0; base < 1024; base += 8)
        for (int t = 0; t < 8; t++) out[base + t] = perm[base + inter[t]];
}

/* crates/kiln-marlin-gemm/src/lib.rs:333-341 (build_scale_perm). */
void oracle_build_scale_perm(int32_t *out /* [64] */) {
    int p = 0;
    for (int i = 0; i < 8; i++)
        for (int j = 0; j < 8; j++) out[p++] = i + 8 * j;
}

/* crates/kiln-marlin-gemm/src/lib.rs:348-357 (build_scale_perm_single). */
void oracle_build_scale_perm_single(int32_t *out /* [32] */) {
    static const int inner[8] = {0, 1, 8, 9, 16, 17, 24, 25};
    int p = 0;
    for (int i = 0; i < 4; i++)
        for (int j = 0; j < 8; j++) out[p++] = 2 * i + inner[j];
}

/* ---- a2: tile transpose + fragment permutation + nibble packing ------------ */

/* crates/kiln-marlin-gemm/src/lib.rs:429-479: q[k,n] (values 0..15) ->
 * packed [k/16, 2n] int32.  Same loop order and temporaries as the reference. */
int oracle_pack_nibbles(const uint8_t *q, int k, int n, int32_t *packed) {
    if (k % 16 || n % 64) return 1;
    int kt = k / 16, nt = n / 16;
    size_t row_len = (size_t)n * 16;
    int32_t *tiled = (int32_t *)malloc(sizeof(int32_t) * kt * row_len);
    int32_t *permuted = (int32_t *)malloc(sizeof(int32_t) * kt * row_len);
    if (!tiled || !permuted) { free(tiled); free(permuted); return 2; }
    for (int kb = 0; kb < kt; kb++)
        for (int nb = 0; nb < nt; nb++)
            for (int tk = 0; tk < 16; tk++)
                for (int tn = 0; tn < 16; tn++) {
                    size_t src = (size_t)(kb * 16 + tk) * n + (nb * 16 + tn);
                    size_t dst = kb * row_len + (size_t)nb * 256 + tk * 16 + tn;
                    tiled[dst] = q[src];
                }
    int32_t perm[1024];
    oracle_build_weight_perm(perm);
    size_t chunks = row_len / 1024;
    for (int r = 0; r < kt; r++)
        for (size_t ch = 0; ch < chunks; ch++) {
            size_t base = r * row_len + ch * 1024;
            for (int i = 0; i < 1024; i++) permuted[base + i] = tiled[base + perm[i]];
        }
    size_t packed_cols = row_len / 8;
    for (int r = 0; r < kt; r++)
        for (size_t c = 0; c < packed_cols; c++) {
            uint32_t acc = 0;
            for (int i = 0; i < 8; i++)
                acc |= ((uint32_t)permuted[r * row_len + c * 8 + i] & 0xFu) << (4 * i);
            packed[r * packed_cols + c] = (int32_t)acc;
        }
    free(tiled);
    free(permuted);
    return 0;
}

/* Independent statement of the same format from the consumer's side: word w of
 * packed row kb holds, for lane = (w%128)/4 and 16-column tile j = w%4 of the
 * 64-column chunk w/128, the eight B-operand elements that lane owns in two
 * mma.m16n8k16 fragments (csrc/marlin_kernel.cu:131-152 dequant order,
 * :442-461 fragment use).  Used to cross-check oracle_pack_nibbles. */
int oracle_unpack_fragment(const int32_t *packed, int k, int n, uint8_t *q) {
    if (k % 16 || n % 64) return 1;
    static const int dr[8] = {0, 8, 0, 8, 1, 9, 1, 9};
    static const int dc[8] = {0, 0, 8, 8, 0, 0, 8, 8};
    int kt = k / 16;
    size_t words = (size_t)2 * n;
    for (int kb = 0; kb < kt; kb++)
        for (size_t w = 0; w < words; w++) {
            uint32_t x = (uint32_t)packed[kb * words + w];
            int chunk = (int)(w / 128), lane = (int)((w % 128) / 4), j = (int)(w % 4);
            int r0 = 2 * (lane % 4), c = lane / 4, nb = chunk * 64 + j * 16;
            for (int i = 0; i < 8; i++)
                q[(size_t)(kb * 16 + r0 + dr[i]) * n + nb + c + dc[i]] = (x >> (4 * i)) & 0xF;
        }
    return 0;
}

/* ---- a3: scale permutation --------------------------------------------------- */

/* crates/kiln-marlin-gemm/src/lib.rs:496-528.  `scales` are f16 bit patterns
 * (the permutation moves values, it never re-rounds them; :488 is exact). */
int oracle_permute_scales(const uint16_t *scales, int num_groups, int n, int groupsize,
                          uint16_t *out) {
    if (groupsize == -1) {
        if (num_groups != 1 || n % 32) return 1;
        int32_t sps[32];
        oracle_build_scale_perm_single(sps);
        for (int sub = 0; sub < n / 32; sub++)
            for (int i = 0; i < 32; i++) out[sub * 32 + i] = scales[sub * 32 + sps[i]];
        return 0;
    }
    if (n % 64) return 1;
    int32_t sp[64];
    oracle_build_scale_perm(sp);
    for (int g = 0; g < num_groups; g++)
        for (int sub = 0; sub < n / 64; sub++)
            for (int i = 0; i < 64; i++)
                out[(size_t)g * n + sub * 64 + i] = scales[(size_t)g * n + sub * 64 + sp[i]];
    return 0;
}

/* ---- a1..a3: the whole reference entry point --------------------------------- */

/* crates/kiln-marlin-gemm/src/lib.rs:370-491 (pack::quantize_and_pack).
 * weight: row-major [k,n] f32.  Outputs: packed [k/16, 2n] i32, permuted
 * scales [k/g, n] f16 bits, dequant [k,n] f32 (unpermuted).  `q_out` (optional)
 * receives the raw nibbles [k,n].  Returns non-zero where the reference asserts. */
int oracle_quantize_and_pack(const float *weight, int k, int n, int groupsize,
                             int32_t *packed, uint16_t *scales_f16, float *dequant,
                             uint8_t *q_out) {
    if (k % 128 || n % 256) return 1;               /* lib.rs:377-378 */
    int g = groupsize == -1 ? k : groupsize;        /* lib.rs:380-384 */
    if (g <= 0 || k % g) return 1;                  /* lib.rs:385 */
    int num_groups = k / g;
    float *scales = (float *)malloc(sizeof(float) * (size_t)num_groups * n);
    uint8_t *q = (uint8_t *)malloc((size_t)k * n);
    uint16_t *sbits = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)num_groups * n);
    if (!scales || !q || !sbits) { free(scales); free(q); free(sbits); return 2; }
    /* 1) scales, lib.rs:393-413 */
    for (int grp = 0; grp < num_groups; grp++)
        for (int col = 0; col < n; col++) {
            float max_abs = 0.0f;
            for (int r = 0; r < g; r++) {
                float v = fabsf(weight[(size_t)(grp * g + r) * n + col]);
                if (v > max_abs) max_abs = v;
            }
            if (max_abs == 0.0f) max_abs = 1.0f;
            float s_f32 = (2.0f * max_abs) / (float)MAX_Q;
            uint16_t hb = f32_to_f16_bits(s_f32);
            sbits[(size_t)grp * n + col] = hb;
            scales[(size_t)grp * n + col] = f16_bits_to_f32(hb);
        }
    /* 2) quantise, lib.rs:416-427: f32 divide, round half away, +8, clamp */
    for (int r = 0; r < k; r++) {
        int grp = r / g;
        for (int col = 0; col < n; col++) {
            float s = scales[(size_t)grp * n + col];
            float rr = roundf(weight[(size_t)r * n + col] / s);
            int32_t raw;
            if (rr != rr) raw = 0;                   /* Rust `as i32`: NaN -> 0, saturating */
            else if (rr >= 2147483648.0f) raw = INT32_MAX;
            else if (rr <= -2147483648.0f) raw = INT32_MIN;
            else raw = (int32_t)rr;
            int64_t shifted = (int64_t)raw + Q_OFFSET;
            if (shifted < 0) shifted = 0;
            if (shifted > MAX_Q) shifted = MAX_Q;
            q[(size_t)r * n + col] = (uint8_t)shifted;
            if (dequant) dequant[(size_t)r * n + col] = (float)((int)shifted - Q_OFFSET) * s;
        }
    }
    /* 3-4) tile, permute, pack */
    int rc = oracle_pack_nibbles(q, k, n, packed);
    /* 5) scale permutation, lib.rs:481-488 */
    if (!rc) rc = oracle_permute_scales(sbits, num_groups, n, groupsize, scales_f16);
    if (q_out) memcpy(q_out, q, (size_t)k * n);
    free(scales); free(q); free(sbits);
    return rc;
}

/* ---- GEMM oracles -------------------------------------------------------------- */

/* The fp32-semantics oracle the tolerance is stated against: exact operand
 * values (bf16 A, (nib-8) * f16 scale), accumulated in f64, returned as f32.
 * a: bf16 bits [m,k]; q: nibbles [k,n]; scales: UNPERMUTED f16 bits [k/g, n]. */
int oracle_gemm_fp64(const uint16_t *a, const uint8_t *q, const uint16_t *scales, int m, int n,
                     int k, int groupsize, float *out) {
    int g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || k % g) return 1;
#pragma omp parallel for schedule(static)
    for (int col = 0; col < n; col++) {
        double *acc = (double *)calloc((size_t)m, sizeof(double));
        for (int r = 0; r < k; r++) {
            double w = (double)((int)q[(size_t)r * n + col] - Q_OFFSET) *
                       (double)f16_bits_to_f32(scales[(size_t)(r / g) * n + col]);
            for (int i = 0; i < m; i++) acc[i] += (double)bf16_bits_to_f32(a[(size_t)i * k + r]) * w;
        }
        for (int i = 0; i < m; i++) out[(size_t)i * n + col] = (float)acc[i];
        free(acc);
    }
    return 0;
}

/* Step (i) of the reference's CPU dequantise-then-matmul path: dequant
 * (nib-8)*s in f32, rounded to bf16, laid out [k,n]
 * (crates/kiln-marlin-gemm/tests/parity.rs:94-101). */
int oracle_dequant_bf16(const uint8_t *q, const uint16_t *scales, int n, int k, int groupsize,
                        uint16_t *w_bf16) {
    int g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || k % g) return 1;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < k; r++)
        for (int col = 0; col < n; col++) {
            float s = f16_bits_to_f32(scales[(size_t)(r / g) * n + col]);
            w_bf16[(size_t)r * n + col] = f32_to_bf16_bits((float)((int)q[(size_t)r * n + col] - Q_OFFSET) * s);
        }
    return 0;
}

/* Steps (ii)-(iii): both operands upcast to f32, f32 GEMM with f32
 * accumulation (kiln's CPU matmul convention,
 * crates/kiln-model/src/lora_loader.rs:233-245), result rounded to bf16.
 * Threads over column blocks; rows of W are walked contiguously. */
int oracle_matmul_bf16(const uint16_t *a, const uint16_t *w_bf16, int m, int n, int k,
                       uint16_t *out_bf16) {
    enum { NB = 256 };
    int nblocks = (n + NB - 1) / NB;
#pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < nblocks; b++) {
        int c0 = b * NB, c1 = c0 + NB > n ? n : c0 + NB;
        float acc[NB];
        float wrow[NB];
        for (int i = 0; i < m; i++) {
            for (int c = 0; c < c1 - c0; c++) acc[c] = 0.0f;
            for (int r = 0; r < k; r++) {
                float av = bf16_bits_to_f32(a[(size_t)i * k + r]);
                const uint16_t *wr = w_bf16 + (size_t)r * n + c0;
                for (int c = 0; c < c1 - c0; c++) wrow[c] = bf16_bits_to_f32(wr[c]);
                for (int c = 0; c < c1 - c0; c++) acc[c] += av * wrow[c];
            }
            for (int c = 0; c < c1 - c0; c++) out_bf16[(size_t)i * n + c0 + c] = f32_to_bf16_bits(acc[c]);
        }
    }
    return 0;
}

/* The whole CPU path in one call (what the benchmark times as the CPU
 * baseline): dequantise to bf16 [k,n], then matmul.  `scratch_w` is a
 * caller-provided k*n uint16 buffer. */
int oracle_w4a16_gemm_cpu(const uint16_t *a, const uint8_t *q, const uint16_t *scales, int m, int n,
                          int k, int groupsize, uint16_t *scratch_w, uint16_t *out_bf16) {
    int rc = oracle_dequant_bf16(q, scales, n, k, groupsize, scratch_w);
    if (rc) return rc;
    return oracle_matmul_bf16(a, scratch_w, m, n, k, out_bf16);
}

/* Number of threads the OpenMP runtime will use (reported as `cores`). */
#ifdef _OPENMP
#include <omp.h>
int oracle_num_threads(void) { return omp_get_max_threads(); }
void oracle_set_num_threads(int n) {
    if (n > 0) omp_set_num_threads(n);
}
#else
int oracle_num_threads(void) { return 1; }
void oracle_set_num_threads(int n) { (void)n; }
#endif
