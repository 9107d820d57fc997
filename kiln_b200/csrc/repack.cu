// Native weight repacker: symmetric int4 quantiser + Marlin tile/fragment packing + scale
// reordering, on the host (multi-threaded inside one matrix) and on the device.
//
// Output is bit-identical to kiln's `pack::quantize_and_pack`
// (kiln-marlin-gemm/src/lib.rs:370-491) but computed directly: no k*n temporaries and no
// 1024-entry gather; every packed word is assembled from the eight weights the consuming lane
// owns (see the layout note in w4a16_common.cuh).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "w4a16_common.cuh"

namespace kiln {
namespace {

constexpr int kMaxQ = 15;    // kiln-marlin-gemm/src/lib.rs:288
constexpr int kQOffset = 8;  // kiln-marlin-gemm/src/lib.rs:289

// (row, col) offsets of nibble i inside a lane's word, relative to (2*(lane%4), lane/4)
__host__ __device__ inline int nib_dr(int i) { return ((i >> 2) & 1) + 8 * (i & 1); }
__host__ __device__ inline int nib_dc(int i) { return 8 * ((i >> 1) & 1); }

// position of natural column `col` in the grouped scale order (lib.rs:333-341):
// out[8i + j] = in[i + 8j] within each 64 columns.
__host__ __device__ inline int scale_group_pos(int col) {
    const int c64 = col & 63;
    return (col & ~63) + 8 * (c64 & 7) + (c64 >> 3);
}

__host__ __device__ inline int quantize_one(float w, float s) {
    // lib.rs:422-423: f32 divide, round half away from zero, +8, clamp to [0,15]
    float r = roundf(w / s);
    // Rust `as i32` saturates and maps NaN to 0
    int raw;
    if (r != r) raw = 0;
    else if (r >= 2147483648.0f) raw = 2147483647;
    else if (r <= -2147483648.0f) raw = -2147483647 - 1;
    else raw = static_cast<int>(r);
    long long shifted = static_cast<long long>(raw) + kQOffset;
    if (shifted < 0) shifted = 0;
    if (shifted > kMaxQ) shifted = kMaxQ;
    return static_cast<int>(shifted);
}

// ---- host ---------------------------------------------------------------------------------

inline uint16_t host_f32_to_f16_bits(float f) {
    const __half h = __float2half_rn(f);  // host path of cuda_fp16: IEEE round-to-nearest-even
    uint16_t b;
    std::memcpy(&b, &h, 2);
    return b;
}
inline float host_f16_bits_to_f32(uint16_t b) {
    __half h;
    std::memcpy(&h, &b, 2);
    return __half2float(h);
}

template <class F>
void parallel_chunks(int chunks, int num_threads, F &&fn) {
    int nt = num_threads > 0 ? num_threads : static_cast<int>(std::thread::hardware_concurrency());
    if (nt < 1) nt = 1;
    nt = std::min(nt, chunks);
    if (nt <= 1) {
        for (int c = 0; c < chunks; ++c) fn(c);
        return;
    }
    std::vector<std::thread> pool;
    pool.reserve(nt);
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([=, &fn] {
            for (int c = t; c < chunks; c += nt) fn(c);
        });
    for (auto &th : pool) th.join();
}

// Packs one 64-column chunk of a 16-row K-tile whose nibbles are in nib[16][64].
inline void pack_tile_host(const uint8_t (*nib)[64], int32_t *out128) {
    for (int lane = 0; lane < 32; ++lane) {
        const int r0 = 2 * (lane & 3), c = lane >> 2;
        for (int j = 0; j < 4; ++j) {
            uint32_t word = 0;
            for (int i = 0; i < 8; ++i)
                word |= static_cast<uint32_t>(nib[r0 + nib_dr(i)][16 * j + c + nib_dc(i)] & 0xF) << (4 * i);
            out128[lane * 4 + j] = static_cast<int32_t>(word);
        }
    }
}

int shape_ok(int k, int n, int groupsize, int *g_out) {
    if (k <= 0 || n <= 0) return KILN_W4A16_ERR_ARG;
    if (k % 128 != 0 || n % 256 != 0) return KILN_W4A16_ERR_PROB_SHAPE;  // lib.rs:377-378
    const int g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || g % 16 != 0 || k % g != 0) return KILN_W4A16_ERR_PROB_SHAPE;  // lib.rs:385
    *g_out = g;
    return 0;
}

}  // namespace
}  // namespace kiln

using namespace kiln;

extern "C" {

void kiln_w4a16_build_weight_perm(int32_t *out) {
    // Derived from the fragment ownership rather than the reference's list construction:
    // output element e = word*8 + nibble of a 1024-element chunk takes the tiled element
    // 256*j + 16*row + col.
    for (int lane = 0; lane < 32; ++lane)
        for (int j = 0; j < 4; ++j)
            for (int i = 0; i < 8; ++i) {
                const int row = 2 * (lane & 3) + nib_dr(i), col = (lane >> 2) + nib_dc(i);
                out[(lane * 4 + j) * 8 + i] = 256 * j + 16 * row + col;
            }
}

void kiln_w4a16_build_scale_perm(int32_t *out) {
    for (int col = 0; col < 64; ++col) out[scale_group_pos(col)] = col;
}

void kiln_w4a16_build_scale_perm_single(int32_t *out) {
    for (int col = 0; col < 32; ++col) out[scale_single_pos(col)] = col;
}

kiln_w4a16_status_t kiln_w4a16_quantize_and_pack_host(const float *weight, int k, int n, int groupsize,
                                                      int32_t *b_packed, uint16_t *scales_f16,
                                                      float *dequant, int num_threads) {
    int g = 0;
    if (int rc = shape_ok(k, n, groupsize, &g)) return rc;
    if (!weight || !b_packed || !scales_f16) return KILN_W4A16_ERR_ARG;
    const int chunks = n / 64, ktiles_per_group = g / 16, num_groups = k / g;
    const size_t row_words = static_cast<size_t>(2) * n;
    parallel_chunks(chunks, num_threads, [&](int ch) {
        const int c0 = ch * 64;
        float s[64];
        uint8_t nib[16][64];
        for (int grp = 0; grp < num_groups; ++grp) {
            // 1) scales for 64 columns of this group (lib.rs:393-413)
            float mx[64];
            for (int c = 0; c < 64; ++c) mx[c] = 0.f;
            for (int r = 0; r < g; ++r) {
                const float *wr = weight + static_cast<size_t>(grp * g + r) * n + c0;
                for (int c = 0; c < 64; ++c) {
                    const float v = std::fabs(wr[c]);
                    if (v > mx[c]) mx[c] = v;
                }
            }
            for (int c = 0; c < 64; ++c) {
                if (mx[c] == 0.f) mx[c] = 1.f;
                const uint16_t hb = host_f32_to_f16_bits((2.0f * mx[c]) / static_cast<float>(kMaxQ));
                s[c] = host_f16_bits_to_f32(hb);
                const int pos = groupsize == -1 ? scale_single_pos(c0 + c) : scale_group_pos(c0 + c);
                scales_f16[static_cast<size_t>(grp) * n + pos] = hb;
            }
            // 2-4) quantise and pack, one 16-row tile at a time
            for (int kt = 0; kt < ktiles_per_group; ++kt) {
                const int kb = grp * ktiles_per_group + kt;
                for (int r = 0; r < 16; ++r) {
                    const size_t off = static_cast<size_t>(kb * 16 + r) * n + c0;
                    for (int c = 0; c < 64; ++c) {
                        const int qv = quantize_one(weight[off + c], s[c]);
                        nib[r][c] = static_cast<uint8_t>(qv);
                        if (dequant) dequant[off + c] = static_cast<float>(qv - kQOffset) * s[c];
                    }
                }
                pack_tile_host(nib, b_packed + static_cast<size_t>(kb) * row_words + ch * 128);
            }
        }
    });
    return KILN_W4A16_OK;
}

kiln_w4a16_status_t kiln_w4a16_repack_host(const uint8_t *q, const uint16_t *scales, int k, int n,
                                           int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                           int num_threads) {
    int g = 0;
    if (k <= 0 || n <= 0) return KILN_W4A16_ERR_ARG;
    if (k % 16 != 0 || n % 64 != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || k % g != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    if (!q || !scales || !b_packed || !scales_perm) return KILN_W4A16_ERR_ARG;
    const int chunks = n / 64, num_groups = k / g;
    const size_t row_words = static_cast<size_t>(2) * n;
    parallel_chunks(chunks, num_threads, [&](int ch) {
        const int c0 = ch * 64;
        uint8_t nib[16][64];
        for (int kb = 0; kb < k / 16; ++kb) {
            for (int r = 0; r < 16; ++r)
                std::memcpy(nib[r], q + static_cast<size_t>(kb * 16 + r) * n + c0, 64);
            pack_tile_host(nib, b_packed + static_cast<size_t>(kb) * row_words + ch * 128);
        }
        for (int grp = 0; grp < num_groups; ++grp)
            for (int c = 0; c < 64; ++c) {
                const int pos = groupsize == -1 ? scale_single_pos(c0 + c) : scale_group_pos(c0 + c);
                scales_perm[static_cast<size_t>(grp) * n + pos] = scales[static_cast<size_t>(grp) * n + c0 + c];
            }
    });
    return KILN_W4A16_OK;
}


// GPTQ checkpoint tensors -> W4A16 layout without dequantising (kiln dequantises GPTQ to bf16 on the CPU,
// crates/kiln-model/src/quantized.rs:70-163, and the Marlin path then re-quantises that).  qweight int32 [k/8, n]
// (nibble i of a word = input row 8*row + i), qzeros int32 [k/g, n/8] (nibble j of a word = output column 8*col + j),
// scales fp16 [k/g, n].  GPTQ's value is (nibble - zero) * scale, this format's is (nibble - 8) * scale: the repack is
// exact when every zero-point is 8, and refused (KILN_W4A16_ERR_PROB_SHAPE, *asymmetric = how many are not) otherwise.
kiln_w4a16_status_t kiln_w4a16_repack_gptq_host(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                                                int k, int n, int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                                uint32_t *asymmetric, int num_threads) {
    if (k <= 0 || n <= 0) return KILN_W4A16_ERR_ARG;
    if (k % 16 != 0 || n % 64 != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    const int g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || k % g != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    if (!qweight || !qzeros || !scales || !b_packed || !scales_perm) return KILN_W4A16_ERR_ARG;
    const int num_groups = k / g;
    uint32_t bad = 0;
    for (size_t i = 0; i < static_cast<size_t>(num_groups) * (n / 8); ++i) {
        const uint32_t z = static_cast<uint32_t>(qzeros[i]);
        for (int j = 0; j < 8; ++j) bad += ((z >> (4 * j)) & 0xF) != static_cast<uint32_t>(kQOffset);
    }
    if (asymmetric) *asymmetric = bad;
    if (bad) return KILN_W4A16_ERR_PROB_SHAPE;
    const int chunks = n / 64;
    const size_t row_words = static_cast<size_t>(2) * n;
    parallel_chunks(chunks, num_threads, [&](int ch) {
        const int c0 = ch * 64;
        uint8_t nib[16][64];
        for (int kb = 0; kb < k / 16; ++kb) {
            for (int r = 0; r < 16; ++r) {
                const int32_t *row = qweight + static_cast<size_t>((kb * 16 + r) / 8) * n + c0;
                const int sh = 4 * ((kb * 16 + r) % 8);
                for (int c = 0; c < 64; ++c) nib[r][c] = static_cast<uint8_t>((static_cast<uint32_t>(row[c]) >> sh) & 0xF);
            }
            pack_tile_host(nib, b_packed + static_cast<size_t>(kb) * row_words + ch * 128);
        }
        for (int grp = 0; grp < num_groups; ++grp)
            for (int c = 0; c < 64; ++c) {
                const int pos = groupsize == -1 ? scale_single_pos(c0 + c) : scale_group_pos(c0 + c);
                scales_perm[static_cast<size_t>(grp) * n + pos] = scales[static_cast<size_t>(grp) * n + c0 + c];
            }
    });
    return KILN_W4A16_OK;
}

}  // extern "C"

// ---- device -------------------------------------------------------------------------------
namespace kiln {
namespace {

template <bool BF16>
__device__ __forceinline__ float load_w(const void *w, size_t idx) {
    if (BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(w)[idx]);
    return static_cast<const float *>(w)[idx];
}

// One thread per column: max |w| over the group, f16 scale, written at its Marlin position.
// grid = (n/128, num_groups), block = 128.  `scales_nat` keeps the natural order for kernel 2.
template <bool BF16>
__global__ void pack_scales_kernel(const void *w, int n, int g, int per_column, uint16_t *scales_perm,
                                   float *scales_nat) {
    const int col = blockIdx.x * blockDim.x + threadIdx.x;
    const int grp = blockIdx.y;
    if (col >= n) return;
    float mx = 0.f;
    for (int r = 0; r < g; ++r) mx = fmaxf(mx, fabsf(load_w<BF16>(w, static_cast<size_t>(grp * g + r) * n + col)));
    if (mx == 0.f) mx = 1.f;
    const __half h = __float2half_rn(__fdiv_rn(2.0f * mx, 15.0f));
    const int pos = per_column ? scale_single_pos(col) : scale_group_pos(col);
    scales_perm[static_cast<size_t>(grp) * n + pos] = __half_as_ushort(h);
    scales_nat[static_cast<size_t>(grp) * n + col] = __half2float(h);
}

// One block per (16-row K-tile, 64-column chunk); thread (lane, j) assembles one packed word.
// grid = (n/64, k/16), block = 128.
template <bool BF16>
__global__ void pack_words_kernel(const void *w, int n, int g, const float *scales_nat, int32_t *b_packed,
                                  float *dequant) {
    __shared__ uint8_t nib[16][64];
    const int ch = blockIdx.x, kb = blockIdx.y, tid = threadIdx.x;
    const int grp = (kb * 16) / g;
    for (int e = tid; e < 16 * 64; e += blockDim.x) {
        const int r = e >> 6, c = e & 63;
        const size_t off = static_cast<size_t>(kb * 16 + r) * n + ch * 64 + c;
        const float s = scales_nat[static_cast<size_t>(grp) * n + ch * 64 + c];
        const float wv = load_w<BF16>(w, off);
        const int qv = quantize_one(wv, s);
        nib[r][c] = static_cast<uint8_t>(qv);
        if (dequant) dequant[off] = __fmul_rn(static_cast<float>(qv - kQOffset), s);
    }
    __syncthreads();
    const int lane = tid >> 2, j = tid & 3;
    const int r0 = 2 * (lane & 3), c = lane >> 2;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        word |= static_cast<uint32_t>(nib[r0 + nib_dr(i)][16 * j + c + nib_dc(i)] & 0xF) << (4 * i);
    b_packed[static_cast<size_t>(kb) * 2 * n + ch * 128 + tid] = static_cast<int32_t>(word);
}

// Grouped mode (128 rows per scale), everything in one pass: one block per (scale group, 64-column chunk) reads its
// 128 x 64 weights once (16-byte loads, 128 contiguous bytes per row), finds the column maxima, writes the 64 fp16
// scales at their Marlin positions and the eight 512-byte packed blocks.  Same arithmetic as the two kernels above.
// grid = (n/64, k/128), block = 256.
template <bool BF16>
__global__ void __launch_bounds__(256) pack_group_kernel(const void *w, int n, uint16_t *scales_perm, int32_t *b_packed, float *dequant) {
    __shared__ float tile[128][65];
    __shared__ float part_max[4][64];
    __shared__ float s_col[64];
    const int ch = blockIdx.x, grp = blockIdx.y, tid = threadIdx.x;
    const size_t row0 = static_cast<size_t>(grp) * 128;
    // 128 rows x 8 pieces of 8 weights
    for (int e = tid; e < 128 * 8; e += 256) {
        const int r = e >> 3, p8 = e & 7;
        const size_t off = (row0 + r) * n + ch * 64 + p8 * 8;
        float v[8];
        if (BF16) {
            const uint4 raw = *reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(w) + off);
            const uint32_t x[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                v[2 * i] = __uint_as_float(x[i] << 16);
                v[2 * i + 1] = __uint_as_float(x[i] & 0xFFFF0000u);
            }
        } else {
            const float4 a = *reinterpret_cast<const float4 *>(static_cast<const float *>(w) + off);
            const float4 b = *reinterpret_cast<const float4 *>(static_cast<const float *>(w) + off + 4);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
            v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) tile[r][p8 * 8 + i] = v[i];
    }
    __syncthreads();
    {
        const int col = tid & 63, part = tid >> 6;
        float mx = 0.f;
        for (int r = 0; r < 32; ++r) mx = fmaxf(mx, fabsf(tile[part * 32 + r][col]));
        part_max[part][col] = mx;
    }
    __syncthreads();
    if (tid < 64) {
        float mx = fmaxf(fmaxf(part_max[0][tid], part_max[1][tid]), fmaxf(part_max[2][tid], part_max[3][tid]));
        if (mx == 0.f) mx = 1.f;
        const __half h = __float2half_rn(__fdiv_rn(2.0f * mx, 15.0f));
        scales_perm[static_cast<size_t>(grp) * n + scale_group_pos(ch * 64 + tid)] = __half_as_ushort(h);
        s_col[tid] = __half2float(h);
    }
    __syncthreads();
    for (int idx = tid; idx < 8 * 128; idx += 256) {
        const int kt = idx >> 7, t128 = idx & 127;
        const int lane = t128 >> 2, j = t128 & 3;
        const int r0 = kt * 16 + 2 * (lane & 3), c = lane >> 2;
        uint32_t word = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int cc = 16 * j + c + nib_dc(i);
            word |= static_cast<uint32_t>(quantize_one(tile[r0 + nib_dr(i)][cc], s_col[cc])) << (4 * i);
        }
        b_packed[(static_cast<size_t>(grp) * 8 + kt) * 2 * n + ch * 128 + t128] = static_cast<int32_t>(word);
    }
    if (dequant) {
        for (int e = tid; e < 128 * 64; e += 256) {
            const int r = e >> 6, c = e & 63;
            const float sc = s_col[c];
            dequant[(row0 + r) * n + ch * 64 + c] = __fmul_rn(static_cast<float>(quantize_one(tile[r][c], sc) - kQOffset), sc);
        }
    }
}

// Already-quantised input: q uint8 [k,n] -> packed words; scales moved to Marlin order.
__global__ void repack_words_kernel(const uint8_t *q, int n, int32_t *b_packed) {
    __shared__ uint8_t nib[16][64];
    const int ch = blockIdx.x, kb = blockIdx.y, tid = threadIdx.x;
    for (int e = tid; e < 16 * 16; e += blockDim.x) {  // 16 rows x 16 uint32 (4 nibble bytes each)
        const int r = e >> 4, c4 = e & 15;
        *reinterpret_cast<uint32_t *>(&nib[r][4 * c4]) =
            *reinterpret_cast<const uint32_t *>(q + static_cast<size_t>(kb * 16 + r) * n + ch * 64 + 4 * c4);
    }
    __syncthreads();
    const int lane = tid >> 2, j = tid & 3;
    const int r0 = 2 * (lane & 3), c = lane >> 2;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        word |= static_cast<uint32_t>(nib[r0 + nib_dr(i)][16 * j + c + nib_dc(i)] & 0xF) << (4 * i);
    b_packed[static_cast<size_t>(kb) * 2 * n + ch * 128 + tid] = static_cast<int32_t>(word);
}

// GPTQ qweight int32 [k/8, n] -> packed words (same gather as above from the two GPTQ words a 16-row tile spans).
__global__ void repack_gptq_words_kernel(const int32_t *qweight, int n, int32_t *b_packed) {
    const int ch = blockIdx.x, kb = blockIdx.y, tid = threadIdx.x;
    const int lane = tid >> 2, j = tid & 3;
    const int r0 = 2 * (lane & 3), c = lane >> 2;
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = r0 + nib_dr(i), col = ch * 64 + 16 * j + c + nib_dc(i);
        const uint32_t src = static_cast<uint32_t>(qweight[static_cast<size_t>(kb * 2 + (r >> 3)) * n + col]);
        word |= ((src >> (4 * (r & 7))) & 0xFu) << (4 * i);
    }
    b_packed[static_cast<size_t>(kb) * 2 * n + ch * 128 + tid] = static_cast<int32_t>(word);
}

// counts the zero-points that are not 8 (one word = eight of them)
__global__ void count_asymmetric_kernel(const int32_t *qzeros, size_t words, uint32_t *count) {
    uint32_t bad = 0;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < words; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t z = static_cast<uint32_t>(qzeros[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) bad += ((z >> (4 * j)) & 0xFu) != static_cast<uint32_t>(kQOffset);
    }
    if (bad) atomicAdd(count, bad);
}

__global__ void permute_scales_kernel(const uint16_t *scales, int n, int per_column, uint16_t *out) {
    const int col = blockIdx.x * blockDim.x + threadIdx.x, grp = blockIdx.y;
    if (col >= n) return;
    const int pos = per_column ? scale_single_pos(col) : scale_group_pos(col);
    out[static_cast<size_t>(grp) * n + pos] = scales[static_cast<size_t>(grp) * n + col];
}

// The GEMM kernels are launched with programmatic stream serialisation and read the packed weights and scales BEFORE
// their grid-dependency wait (weights normally never depend on the kernel before a GEMM).  A GEMM enqueued right after a
// device pack would break that assumption, so every device pack entry point ends with this ordinary launch: it starts
// only when the pack kernels have completed and flushed, and it is what the next kernel's early part overlaps with.
__global__ void pack_fence_kernel() {}

}  // namespace
}  // namespace kiln

extern "C" {

kiln_w4a16_status_t kiln_w4a16_quantize_and_pack_device(const void *weight, int weight_is_bf16, int k, int n,
                                                        int groupsize, int32_t *b_packed,
                                                        uint16_t *scales_f16, float *dequant, void *stream) {
    int g = 0;
    if (int rc = shape_ok(k, n, groupsize, &g)) return rc;
    if (!weight || !b_packed || !scales_f16) return KILN_W4A16_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int num_groups = k / g;
    if (groupsize == 128 && (reinterpret_cast<uintptr_t>(weight) & 15) == 0) {  // (n is a multiple of 64: rows stay 16-byte aligned)
        const dim3 grid(n / 64, k / 128);
        if (weight_is_bf16)
            pack_group_kernel<true><<<grid, 256, 0, st>>>(weight, n, scales_f16, b_packed, dequant);
        else
            pack_group_kernel<false><<<grid, 256, 0, st>>>(weight, n, scales_f16, b_packed, dequant);
        pack_fence_kernel<<<1, 32, 0, st>>>();
        note_launch(2);
        return record_cuda_error(cudaGetLastError());
    }
    float *scales_nat = nullptr;  // natural-order f32 scales, scratch for the second kernel
    if (int rc = record_cuda_error(cudaMallocAsync(&scales_nat, sizeof(float) * num_groups * n, st))) return rc;
    const dim3 g1(n / 128, num_groups), g2(n / 64, k / 16);
    if (weight_is_bf16) {
        pack_scales_kernel<true><<<g1, 128, 0, st>>>(weight, n, g, groupsize == -1, scales_f16, scales_nat);
        pack_words_kernel<true><<<g2, 128, 0, st>>>(weight, n, g, scales_nat, b_packed, dequant);
    } else {
        pack_scales_kernel<false><<<g1, 128, 0, st>>>(weight, n, g, groupsize == -1, scales_f16, scales_nat);
        pack_words_kernel<false><<<g2, 128, 0, st>>>(weight, n, g, scales_nat, b_packed, dequant);
    }
    pack_fence_kernel<<<1, 32, 0, st>>>();
    note_launch(3);
    int rc = record_cuda_error(cudaGetLastError());
    const int rc2 = record_cuda_error(cudaFreeAsync(scales_nat, st));
    return rc ? rc : rc2;
}

kiln_w4a16_status_t kiln_w4a16_repack_device(const uint8_t *q, const uint16_t *scales, int k, int n,
                                             int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                             void *stream) {
    if (k <= 0 || n <= 0) return KILN_W4A16_ERR_ARG;
    if (k % 16 != 0 || n % 64 != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    const int g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || k % g != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    if (!q || !scales || !b_packed || !scales_perm) return KILN_W4A16_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(q) & 3) != 0) return KILN_W4A16_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    repack_words_kernel<<<dim3(n / 64, k / 16), 128, 0, st>>>(q, n, b_packed);
    permute_scales_kernel<<<dim3((n + 127) / 128, k / g), 128, 0, st>>>(scales, n, groupsize == -1, scales_perm);
    pack_fence_kernel<<<1, 32, 0, st>>>();
    note_launch(3);
    return record_cuda_error(cudaGetLastError());
}

// Device variant of kiln_w4a16_repack_gptq_host.  The symmetry check cannot refuse before the launch without a
// synchronisation, so it reports: *asymmetric (a DEVICE uint32, may be NULL) receives the number of zero-points that are
// not 8; the caller reads it (stream-ordered) and discards the output if it is not 0.
kiln_w4a16_status_t kiln_w4a16_repack_gptq_device(const int32_t *qweight, const int32_t *qzeros, const uint16_t *scales,
                                                  int k, int n, int groupsize, int32_t *b_packed, uint16_t *scales_perm,
                                                  uint32_t *asymmetric, void *stream) {
    if (k <= 0 || n <= 0) return KILN_W4A16_ERR_ARG;
    if (k % 16 != 0 || n % 64 != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    const int g = groupsize == -1 ? k : groupsize;
    if (g <= 0 || k % g != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    if (!qweight || !qzeros || !scales || !b_packed || !scales_perm) return KILN_W4A16_ERR_ARG;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned launches = 3;
    if (asymmetric) {
        if (int rc = record_cuda_error(cudaMemsetAsync(asymmetric, 0, sizeof(uint32_t), st))) return rc;
        const size_t words = static_cast<size_t>(k / g) * (n / 8);
        count_asymmetric_kernel<<<static_cast<unsigned>((words + 255) / 256 > 1024 ? 1024 : (words + 255) / 256), 256, 0, st>>>(
            qzeros, words, asymmetric);
        ++launches;
    }
    repack_gptq_words_kernel<<<dim3(n / 64, k / 16), 128, 0, st>>>(qweight, n, b_packed);
    permute_scales_kernel<<<dim3((n + 127) / 128, k / g), 128, 0, st>>>(scales, n, groupsize == -1, scales_perm);
    pack_fence_kernel<<<1, 32, 0, st>>>();
    note_launch(launches);
    return record_cuda_error(cudaGetLastError());
}

}  // extern "C"
