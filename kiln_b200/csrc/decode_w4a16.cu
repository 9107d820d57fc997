// Decode-shape W4A16 GEMM for sm_100a: C[m,n] = A[m,k] * dequant(B)[k,n], m small.
//
// Replaces the reference's `Marlin<256,1,8,8,4,8>` path
// (kiln-marlin-gemm/csrc/marlin_kernel.cu:197-700) with a different decomposition:
//
//  * HBM streaming, GEMV-like.  The unit of work is one 4 KB run of the packed matrix: one 64-column chunk
//    x one 128-row scale group = eight 512-byte rows, 16 bytes per lane each.  Every warp streams its own
//    units straight into registers and keeps eight 16-byte loads per lane in flight: as soon as a register
//    is consumed the load of the same row of the next unit is issued into it.  There is no producer warp,
//    no shared-memory ring and no barrier in the stream, so the bytes in flight per SM are simply
//    (resident warps) x 4 KB, CTAs are small (the next kernel's CTAs move in as this kernel's drain) and
//    the first loads leave before the previous kernel in the stream has finished (programmatic dependent
//    launch; only the activations and the output wait for it).
//  * int4 -> fp16 in registers with five integer instructions per packed word (eight weights): `lop3` ORs
//    the nibbles at bits 0..3 into the mantissa of 1024.0 (value 1024 + nib) and the nibbles at bits 4..7,
//    where they sit, into the mantissa of 64.0, whose unit in the last place is 1/16 (value 64 + nib); one
//    shift by 8 brings the other two nibble pairs into the same positions.  The activations are converted
//    bf16 -> fp16 once when a CTA stages them (the reference kernel is fp16 on both sides,
//    kiln-marlin-gemm/src/lib.rs:169), products are exact and accumulate in fp32.
//  * the offsets (1024 + 8, 64 + 8) are removed per 128-K group by one extra MMA per K-tile against a constant
//    fragment.
//  * up to 8 rows: the MMA is issued transposed (weights are the 16x16 operand, one MMA per packed word);
//    9..16 rows: activations are the 16x16 operand, two MMAs per packed word.
//  * the fp16 group scale is applied once per 128-K group to the fp32 partial sums (exact scale).
//  * split-K without global scratch: K is split over teams of warps inside a CTA and over the CTAs of a
//    thread-block cluster; partial tiles meet in (distributed) shared memory and are summed in a fixed
//    order, so results are bit-reproducible.  The cluster exchange is `st.async` into the owner's shared memory,
//    counted on the owner's mbarrier: a CTA goes on when its own slots are full, not when the whole cluster is done.
//  * the waits are `bar.sync`, one cluster barrier at the start (both reached by every thread on every path),
//    `griddepcontrol.wait`, and the wait on that mbarrier, which is bounded in time and reports through a status word.
#include <algorithm>

#include "w4a16_common.cuh"
#include "w4a16_async.cuh"

namespace kiln {
namespace {

constexpr int kMaxProblems = 8;  // GEMMs one launch may cover (kiln_w4a16_gemm_bf16_grouped)

// One GEMM of a launch.  A launch covers up to kMaxProblems independent GEMMs that share the decomposition
// (cluster size, warps per CTA) and differ in everything else; blockIdx.y runs over the column blocks of all of them.
struct DecodeProblem {
    const __nv_bfloat16 *A;
    const uint4 *B;  // packed weights as 16-byte pieces: [k/16][n/64][32 lanes]
    const __half *S;
    __nv_bfloat16 *C;
    const float *lora_t;           // fp32 [m, lora_r] = scale * x * A^T, or null: no LoRA delta
    const __nv_bfloat16 *lora_b;   // bf16 [n, lora_r]
    int m, n, k;
    int groups;          // k / 128
    int groups_per_cta;  // K groups owned by one CTA of the cluster
    int pass_groups;     // K groups whose activations are staged in shared memory at a time
    int per_column;      // groupsize == -1: one scale row, applied at the end
    int a_pitch;         // bytes per staged activation row (pass_groups*256 + 16)
    int y0;              // first blockIdx.y of this problem
    int lora_r;          // LoRA rank (multiple of 8, 0 = none)
    int swiglu;          // columns hold gate and up interleaved in runs of 32; C is [m, n/2] = silu(gate) * up
};

struct DecodeParams {
    DecodeProblem prob[kMaxProblems];
    int count;
    int warps_n, warps_k;
    int red_pitch;          // floats per reduction row (warps_n*64 + 4 or 8)
    int off_red, off_recv, off_lora, off_mbar;  // shared-memory carve-up (bytes from the 128-byte aligned base)
    int ppr_shift;          // log2 of the output pairs (two adjacent columns) per row of a CTA = 5 + log2(warps_n)
    int own_cols;           // receive slots per row owned by one rank of the cluster
    uint32_t own_magic;     // ceil(2^32 / own_cols): x / own_cols = umulhi(x, own_magic) for the small x used here
    int own_items;          // SwiGLU: (gate pair, up pair) items per row owned by one rank = own_cols / 2
    uint32_t item_magic;    // ceil(2^32 / own_items)
};

constexpr uint32_t kLoMask = 0x000F000Fu, kHiMask = 0x00F000F0u;
constexpr uint32_t kMagicLo = 0x64006400u;   // fp16x2 {1024, 1024}: ulp 1, a nibble at bits 0..3 adds nib
constexpr uint32_t kMagicHi = 0x54005400u;   // fp16x2 {64, 64}: ulp 1/16, a nibble at bits 4..7 adds nib
constexpr uint32_t kNegOffLo = 0xE408E408u;  // fp16x2 {-1032, -1032}
constexpr uint32_t kNegOffHi = 0xD480D480u;  // fp16x2 {-72, -72}

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float half_lo(uint32_t w) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w & 0xFFFFu)));
}
__device__ __forceinline__ float half_hi(uint32_t w) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(w >> 16)));
}

// Two bf16 (one 32-bit word) -> two fp16, round to nearest (exact inside the fp16 range).
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t x) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(__uint_as_float(x & 0xFFFF0000u)), "f"(__uint_as_float(x << 16)));
    return r;
}

// The four fp16x2 registers of one packed word: f[0] col c, K 2qd..2qd+1; f[1] col c+8, same K;
// f[2] col c, K 2qd+8..2qd+9; f[3] col c+8, K 2qd+8..2qd+9.  f[0], f[1] carry +1024, f[2], f[3] carry +64.
__device__ __forceinline__ void dequant_word(uint32_t x, uint32_t (&f)[4]) {
    const uint32_t y = x >> 8;
    f[0] = lop3_and_or(x, kLoMask, kMagicLo);
    f[2] = lop3_and_or(x, kHiMask, kMagicHi);
    f[1] = lop3_and_or(y, kLoMask, kMagicLo);
    f[3] = lop3_and_or(y, kHiMask, kMagicHi);
}

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <int NB>
struct Acc;  // per-lane accumulators of one 64-column chunk

// Up to 8 batch rows, transposed MMA: t[j][i] is column 16j + c + 8*(i/2), batch row 2qd + (i%2).
template <>
struct Acc<1> {
    float t[4][4];
};
// 9..16 batch rows: t[n8][i] is column 8*n8 + 2qd + (i%2), batch row c + 8*(i/2).
template <>
struct Acc<2> {
    float t[8][4];
};

#ifndef KILN_DECODE_JS1
#define KILN_DECODE_JS1 2  // 16-column tiles per sweep over the K-tiles of a unit, up to 8 rows
#endif
#ifndef KILN_DECODE_LB1
#define KILN_DECODE_LB1 640  // most threads of a CTA, up to 8 rows: 640 caps the kernel at 96 registers (20 warps per SM)
#endif
#ifndef KILN_DECODE_JS2
#define KILN_DECODE_JS2 2  // the same for 9..16 rows
#endif

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int j) { return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w)); }

// One unit (8 K-tiles of one 64-column chunk) for one warp, up to 8 batch rows.  `w` holds the unit's eight
// 16-byte pieces.  The unit is processed in sweeps over its K-tiles, JS 16-column tiles at a time (fewer
// partial sums live at once); in the last sweep each piece is replaced by the same row of the next unit as
// soon as it has been read.
template <int JS>
__device__ __forceinline__ void compute_unit_t(uint4 (&w)[8], const uint4 *next, uint32_t kt_stride, bool more,
                                               const uint4 sc, uint32_t a_addr, Acc<1> &acc) {
    float corr[4] = {0.f, 0.f, 0.f, 0.f};
    const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int j0 = 0; j0 < 4; j0 += JS) {
        float g[JS][4];
#pragma unroll
        for (int j = 0; j < JS; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) g[j][i] = 0.f;
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
            const uint4 x = w[kt];
            if (j0 + JS == 4 && more) w[kt] = ld_stream_v4(next + kt * kt_stride);
            uint32_t b0, b1;
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(a_addr + kt * 32));
#pragma unroll
            for (int j = 0; j < JS; ++j) {
                uint32_t f[4];
                dequant_word(word_of(x, j0 + j), f);
                mma_f16_16816(g[j], f[0], f[1], f[2], f[3], b0, b1);
            }
            if (j0 == 0) mma_f16_16816(corr, kNegOffLo, kNegOffLo, kNegOffHi, kNegOffHi, b0, b1);
        }
#pragma unroll
        for (int j = 0; j < JS; ++j) {
            const float s0 = half_lo(sw[j0 + j]), s1 = half_hi(sw[j0 + j]);  // columns 16j + c, 16j + c + 8
            acc.t[j0 + j][0] = fmaf(s0, g[j][0] + corr[0], acc.t[j0 + j][0]);
            acc.t[j0 + j][1] = fmaf(s0, g[j][1] + corr[1], acc.t[j0 + j][1]);
            acc.t[j0 + j][2] = fmaf(s1, g[j][2] + corr[0], acc.t[j0 + j][2]);
            acc.t[j0 + j][3] = fmaf(s1, g[j][3] + corr[1], acc.t[j0 + j][3]);
        }
    }
}

// The same for 9..16 batch rows: activations are the 16x16 operand, every packed word feeds two MMAs
// (columns 16j..16j+7 and 16j+8..16j+15).
template <int JS>
__device__ __forceinline__ void compute_unit_s(uint4 (&w)[8], const uint4 *next, uint32_t kt_stride, bool more,
                                               const uint4 sc0, const uint4 sc1, uint32_t a_addr, Acc<2> &acc) {
    // accumulator columns of this lane are 8t + 2qd + e; their scales sit at 16qd + 8e + t of the chunk's
    // scale order: sc0 holds e = 0, sc1 holds e = 1, eight values each.
    const uint32_t s0w[4] = {sc0.x, sc0.y, sc0.z, sc0.w}, s1w[4] = {sc1.x, sc1.y, sc1.z, sc1.w};
    float corr[4] = {0.f, 0.f, 0.f, 0.f};  // [0], [1]: batch row c; [2], [3]: row c + 8 (every column the same)
#pragma unroll
    for (int j0 = 0; j0 < 4; j0 += JS) {
        float g[2 * JS][4];
#pragma unroll
        for (int t = 0; t < 2 * JS; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) g[t][i] = 0.f;
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) {
            const uint4 x = w[kt];
            if (j0 + JS == 4 && more) w[kt] = ld_stream_v4(next + kt * kt_stride);
            uint32_t a[4];
            ldmatrix_x4(a, a_addr + kt * 32);
#pragma unroll
            for (int j = 0; j < JS; ++j) {
                uint32_t f[4];
                dequant_word(word_of(x, j0 + j), f);
                mma_f16_16816(g[2 * j], a[0], a[1], a[2], a[3], f[0], f[2]);
                mma_f16_16816(g[2 * j + 1], a[0], a[1], a[2], a[3], f[1], f[3]);
            }
            if (j0 == 0) mma_f16_16816(corr, a[0], a[1], a[2], a[3], kNegOffLo, kNegOffHi);
        }
#pragma unroll
        for (int tt = 0; tt < 2 * JS; ++tt) {
            const int t = 2 * j0 + tt;
            const float s0 = (t & 1) ? half_hi(s0w[t >> 1]) : half_lo(s0w[t >> 1]);
            const float s1 = (t & 1) ? half_hi(s1w[t >> 1]) : half_lo(s1w[t >> 1]);
            acc.t[t][0] = fmaf(s0, g[tt][0] + corr[0], acc.t[t][0]);
            acc.t[t][1] = fmaf(s1, g[tt][1] + corr[0], acc.t[t][1]);
            acc.t[t][2] = fmaf(s0, g[tt][2] + corr[2], acc.t[t][2]);
            acc.t[t][3] = fmaf(s1, g[tt][3] + corr[2], acc.t[t][3]);
        }
    }
}


// Set (never cleared by a kernel) when a CTA gave up waiting for the split-K partial sums of its cluster peers;
// kiln_w4a16_check_device_status reads and clears it.  A static word, so that no launch path allocates for it.
__device__ uint32_t g_decode_status;

// Store a float2 into a peer's shared memory; its 8 bytes count on the peer's mbarrier when they have landed.
__device__ __forceinline__ void st_async_f2(uint32_t cluster_addr, float2 v, uint32_t cluster_mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1,%2}, [%3];" ::"r"(cluster_addr),
                 "f"(v.x), "f"(v.y), "r"(cluster_mbar)
                 : "memory");
}

// Wait for phase 0 of this CTA's exchange mbarrier.  Bounded in wall-clock time: a peer that never delivers makes
// the CTA record 0x800 in the status word and leave without writing C.
__device__ __forceinline__ bool mbar_wait_decode(uint32_t bar) {
    if (mbar_try_wait(bar, 0)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, 0)) return true;
        if ((i & 15) == 15 && global_ns() - t0 > kWaitLimitNs) break;
    }
    atomicCAS(&g_decode_status, 0u, 0x800u);
    return false;
}

constexpr uint4 kOnesF16 = {0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u};

// grid = (cluster_k, sum over problems of n / (64*warps_n), ceil(max m / (8*NB))), cluster = (cluster_k, 1, 1),
// block = 32 * warps_n * warps_k: warp wk*warps_n + wn streams chunk wn of the groups i with i % warps_k == wk.
// MULTI: the launch covers several GEMMs (the lookup below and the indexed parameter reads cost a single large GEMM a few
// per cent, so single-GEMM launches use the other instance).
template <int NB, bool MULTI>
__global__ void __launch_bounds__(NB == 1 ? KILN_DECODE_LB1 : 512, 1) w4a16_decode_kernel(const __grid_constant__ DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    uint8_t *base_gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sA = base;

    pdl_launch_dependents();
    constexpr int kRows = 8 * NB;
    // which GEMM of the launch this CTA works on (every CTA of a cluster shares blockIdx.y and .z)
    int pi = 0;
    if (MULTI) {
#pragma unroll
        for (int i = 1; i < kMaxProblems; ++i)
            if (i < p.count && static_cast<int>(blockIdx.y) >= p.prob[i].y0) pi = i;
    }
    const DecodeProblem &q = p.prob[pi];
    if (static_cast<int>(blockIdx.z) * kRows >= q.m) return;  // a GEMM with fewer rows than the tallest of the launch
    Acc<NB> acc;
#pragma unroll
    for (int j = 0; j < 4 * NB; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc.t[j][i] = 0.f;
    {  // ---- streaming part: its coordinates and pointers go out of scope before the reduction ----
    const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nthreads = blockDim.x;
    const int m0 = blockIdx.z * kRows;
    const int m_valid = min(kRows, q.m - m0);
    // A CTA may only be written through distributed shared memory once it is running: every CTA of the cluster
    // announces itself here and checks the others just before the first remote store, long after.  Before it does,
    // it arms the mbarrier that counts the bytes of the split-K exchange it will receive: one float2 per valid row
    // and owned column pair from every rank of the cluster, itself included.
    if (csize > 1) {
        if (tid == 0) {
            const int ppr = 1 << p.ppr_shift;
            const int mine = q.swiglu ? 2 * min(p.own_items, (ppr >> 1) - static_cast<int>(rank) * p.own_items)
                                      : min(p.own_cols, ppr - static_cast<int>(rank) * p.own_cols);
            mbar_init(base + p.off_mbar, 1);
            mbar_init_fence();
            mbar_arrive_expect_tx(base + p.off_mbar, csize * m_valid * max(mine, 0) * 8);
        }
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    }

    const int wn = warp % p.warps_n, wk = warp / p.warps_n;
    const int chunk = (static_cast<int>(blockIdx.y) - q.y0) * p.warps_n + wn;
    const int gc0 = min(q.groups, static_cast<int>(rank) * q.groups_per_cta);
    const int gc1 = min(q.groups, gc0 + q.groups_per_cta);
    const int nst = gc1 - gc0;  // K groups of this CTA
    const int qd = lane & 3, c = lane >> 2;

    // ---- this warp's stream: local groups wk, wk + warps_k, ... of chunk `chunk` ----
    const uint32_t chunks = static_cast<uint32_t>(q.n >> 6);
    const uint32_t kt_stride = chunks * 32;                // 16-byte pieces between K-tiles
    const uint32_t unit_stride = kt_stride * 8 * p.warps_k;  // ... between this warp's units
    const uint4 *wptr = q.B + (static_cast<size_t>(gc0 + wk) * 8 * chunks + chunk) * 32 + lane;
    // scales of a unit: NB = 1 needs the 16 bytes at position 8c of the chunk's scale order (columns c + 8t),
    // NB = 2 the 32 bytes at 16qd (columns 8t + 2qd and 8t + 2qd + 1)
    const uint32_t s_unit_stride = static_cast<uint32_t>(q.n) * p.warps_k / 8;
    const uint4 *sptr = reinterpret_cast<const uint4 *>(q.S + static_cast<size_t>(gc0 + wk) * q.n + chunk * 64) +
                        (NB == 1 ? c : 2 * qd);
    uint4 w[8];
    uint4 sc0 = kOnesF16, sc1 = kOnesF16;
    int gl = wk;  // local group of the unit in flight
    // Weights never depend on the previous kernel: the first unit is requested before waiting for it.
    if (gl < nst) {
#pragma unroll
        for (int kt = 0; kt < 8; ++kt) w[kt] = ld_stream_v4(wptr + kt * kt_stride);
        if (!q.per_column) {
            sc0 = ld_stream_v4(sptr);
            if (NB == 2) sc1 = ld_stream_v4(sptr + 1);
        }
    }
    // LoRA: the rows of B^T for this CTA's columns are weights too; they land in shared memory asynchronously
    if (q.lora_r) {
        const int ppb = q.lora_r >> 3;  // 16-byte pieces per row of lora_b
        const int cols = 64 * p.warps_n;
        const __nv_bfloat16 *src = q.lora_b + static_cast<size_t>(chunk - wn) * 64 * q.lora_r;
        for (int idx = tid; idx < cols * ppb; idx += nthreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(base + p.off_lora + idx * 16), "l"(src + idx * 8) : "memory");
    }

    // lane-constant part of the ldmatrix address.  NB = 1 (x2): lanes 0-7 address rows 0-7 at K+0, lanes 8-15 the
    // same rows at K+8.  NB = 2 (x4): rows 0-7 / 8-15 at K+0 for lanes 0-7 / 8-15, the same at K+8 for lanes 16-31.
    // Only the valid rows are staged: rows past m read the last valid row again (their products land in
    // accumulator rows that are never stored).
    uint32_t a_lane;
    if (NB == 1) {
        a_lane = sA + static_cast<uint32_t>(min(lane & 7, m_valid - 1)) * q.a_pitch + static_cast<uint32_t>((lane >> 3) & 1) * 16u;
    } else {
        a_lane = sA + static_cast<uint32_t>(min((lane & 7) + ((lane >> 3) & 1) * 8, m_valid - 1)) * q.a_pitch +
                 static_cast<uint32_t>(lane >> 4) * 16u;
    }

    // Activation staging.  The addresses of a thread's first 16-byte piece are formed here, before the wait, so that
    // after it only load -> convert -> store -> barrier remain.
    const int ppr_a = min(q.pass_groups, nst) * 16;  // 16-byte pieces per row in the first pass
    const __nv_bfloat16 *a_base = q.A + static_cast<size_t>(m0) * q.k + static_cast<size_t>(gc0) * kGroup;
    const uint4 *a_src0;
    uint32_t a_dst0;
    {
        const int r0 = m_valid == 1 ? 0 : tid / max(ppr_a, 1);
        const int c0 = tid - r0 * ppr_a;
        a_src0 = reinterpret_cast<const uint4 *>(a_base + static_cast<size_t>(r0) * q.k + c0 * 8);
        a_dst0 = sA + r0 * q.a_pitch + c0 * 16;
    }
    auto convert_store = [](uint32_t dst, const uint4 &v) {
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(bf16x2_to_f16x2(v.x)), "r"(bf16x2_to_f16x2(v.y)),
                     "r"(bf16x2_to_f16x2(v.z)), "r"(bf16x2_to_f16x2(v.w))
                     : "memory");
    };

    // Everything below reads A or writes C: order it after the previous kernel in the stream.
    pdl_wait();
    if (q.lora_r) {  // scale * x * A^T of this CTA's rows (written by the kernel before this one)
        const int pieces = m_valid * (q.lora_r >> 2);
        const float *src = q.lora_t + static_cast<size_t>(m0) * q.lora_r;
        const uint32_t dst = base + p.off_lora + 64 * p.warps_n * q.lora_r * 2;
        for (int idx = tid; idx < pieces; idx += nthreads)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + idx * 16), "l"(src + idx * 4) : "memory");
    }

    for (int pg0 = 0; pg0 < nst; pg0 += q.pass_groups) {
        const int plen = min(q.pass_groups, nst - pg0);
        if (pg0 > 0) __syncthreads();  // everyone is done with the previous pass' activations
        // ---- stage A[m0 .. m0+m_valid, (gc0+pg0)*128 .. +plen*128) as fp16 ----
        // A thread's first piece of the first pass goes load -> convert -> store (shortest path: its addresses were
        // formed before the wait).  Any further pieces land raw through 16-byte asynchronous copies, all in flight at
        // once, and are then converted in place by the thread that copied them.
        {
            const int ppr = plen * 16;  // 16-byte pieces per row
            const int total = m_valid * ppr;
            const int first = pg0 == 0 ? tid + nthreads : tid;
            const __nv_bfloat16 *a_src = a_base + static_cast<size_t>(pg0) * kGroup;
            for (int idx = first; idx < total; idx += nthreads) {
                const int r = idx / ppr, pc = idx - r * ppr;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sA + r * q.a_pitch + pc * 16),
                             "l"(a_src + static_cast<size_t>(r) * q.k + pc * 8)
                             : "memory");
            }
            if (pg0 == 0 && tid < total) convert_store(a_dst0, ld_cg_v4(a_src0));
            if (first < total) {
                asm volatile("cp.async.wait_all;" ::: "memory");
                for (int idx = first; idx < total; idx += nthreads) {
                    const int r = idx / ppr, pc = idx - r * ppr;
                    const uint32_t addr = sA + r * q.a_pitch + pc * 16;
                    convert_store(addr, lds_v4(addr));
                }
            }
        }
        __syncthreads();
        // ---- this warp's units of the pass ----
        for (; gl < pg0 + plen; gl += p.warps_k) {
            const bool more = gl + p.warps_k < nst;
            const uint4 *next = wptr + unit_stride;
            const uint32_t a_addr = a_lane + static_cast<uint32_t>(gl - pg0) * 256u;
            if constexpr (NB == 1)
                compute_unit_t<KILN_DECODE_JS1>(w, next, kt_stride, more, sc0, a_addr, acc);
            else
                compute_unit_s<KILN_DECODE_JS2>(w, next, kt_stride, more, sc0, sc1, a_addr, acc);
            wptr = next;
            sptr += s_unit_stride;
            // the next unit's scales are needed only after its eight K-tiles: request them now
            if (more && !q.per_column) {
                sc0 = ld_stream_v4(sptr);
                if (NB == 2) sc1 = ld_stream_v4(sptr + 1);
            }
        }
    }
    }  // streaming part
    // ---- this warp's partial tile -> shared memory ----
    // Thread and block coordinates are read again here (volatile reads cannot be merged with the earlier ones), so
    // that nothing but the accumulators has to stay in registers across the streaming loop.
    uint32_t tid_v, by_v, bz_v;
    asm volatile("mov.u32 %0, %%tid.x;" : "=r"(tid_v));
    asm volatile("mov.u32 %0, %%ctaid.y;" : "=r"(by_v));
    asm volatile("mov.u32 %0, %%ctaid.z;" : "=r"(bz_v));
    const int tid = static_cast<int>(tid_v), lane = tid & 31, warp = tid >> 5;
    const int qd = lane & 3, c = lane >> 2;
    const int wn = warp % p.warps_n, wk = warp / p.warps_n;
    const int m0 = static_cast<int>(bz_v) * kRows;
    const int m_valid = min(kRows, q.m - m0);
    const int nthreads = blockDim.x;
    const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
    float *sRed = reinterpret_cast<float *>(base_gen + p.off_red);
    {
        float *mine = sRed + static_cast<size_t>(wk) * kRows * p.red_pitch + wn * 64;
        if constexpr (NB == 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = 2 * qd + (i & 1);
                    if (row < m_valid) mine[row * p.red_pitch + 16 * j + c + 8 * (i >> 1)] = acc.t[j][i];
                }
        } else {
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int col = 8 * t + 2 * qd;
                if (c < m_valid) *reinterpret_cast<float2 *>(mine + c * p.red_pitch + col) = make_float2(acc.t[t][0], acc.t[t][1]);
                if (c + 8 < m_valid)
                    *reinterpret_cast<float2 *>(mine + (c + 8) * p.red_pitch + col) = make_float2(acc.t[t][2], acc.t[t][3]);
            }
        }
    }
    if (q.lora_r) asm volatile("cp.async.wait_all;" ::: "memory");  // this thread's pieces of lora_b and lora_t
    __syncthreads();

    // ---- reduction over the K-teams of the CTA, then over the CTAs of the cluster -----------
    // An output pair is two adjacent columns of one row.  The pairs of a row are dealt to the cluster ranks in
    // contiguous slices (SwiGLU: slices of items, an item being a gate pair and the up pair 32 columns after it, so
    // that both meet in one rank).  Every CTA sums its K-teams and pushes each pair into the owning rank's receive
    // buffer, slot [sender rank][row][slot of the pair], with stores that count their bytes on the owner's mbarrier;
    // once its slots are full the owner adds them in rank order, finishes the values (per-column scale, LoRA delta,
    // SwiGLU) and writes C.  Everything here is a chain of
    // dependent instructions in few threads, so it avoids divisions and keeps the shared-memory loads of a sum
    // independent of each other.
    const int ppr_shift = p.ppr_shift, ppr = 1 << ppr_shift;
    const int n0 = (static_cast<int>(by_v) - q.y0) * (2 * ppr);  // first column of this CTA within its GEMM
    const size_t team_stride = static_cast<size_t>(kRows) * p.red_pitch;
    auto team_sum = [&](int row, int cp) {
        const float *src = sRed + row * p.red_pitch + 2 * cp;
        float2 v = *reinterpret_cast<const float2 *>(src);
#pragma unroll 4
        for (int t = 1; t < p.warps_k; ++t) {
            const float2 u = *reinterpret_cast<const float2 *>(src + t * team_stride);
            v.x += u.x;
            v.y += u.y;
        }
        return v;
    };
    // complete sums of a pair -> final values: per-column scale, then the LoRA delta of the two columns
    auto finish_pair = [&](int row, int cp, float2 v) {
        const int col = n0 + 2 * cp;
        if (q.per_column) {
            const int pos = scale_single_pos(col);  // col is even: col+1 sits at pos+1
            v.x *= __half2float(q.S[pos]);
            v.y *= __half2float(q.S[pos + 1]);
        }
        if (q.lora_r) {
            const uint4 *b0 = reinterpret_cast<const uint4 *>(base_gen + p.off_lora + static_cast<size_t>(2 * cp) * q.lora_r * 2);
            const uint4 *b1 = b0 + (q.lora_r >> 3);
            const float4 *t = reinterpret_cast<const float4 *>(base_gen + p.off_lora + 64 * p.warps_n * q.lora_r * 2 +
                                                               static_cast<size_t>(row) * q.lora_r * 4);
            float d0 = 0.f, d1 = 0.f;
            for (int j = 0; j < (q.lora_r >> 3); ++j) {
                const uint4 x0 = b0[j], x1 = b1[j];
                const float4 ta = t[2 * j], tb = t[2 * j + 1];
                d0 += ta.x * __uint_as_float(x0.x << 16) + ta.y * __uint_as_float(x0.x & 0xFFFF0000u) +
                      ta.z * __uint_as_float(x0.y << 16) + ta.w * __uint_as_float(x0.y & 0xFFFF0000u) +
                      tb.x * __uint_as_float(x0.z << 16) + tb.y * __uint_as_float(x0.z & 0xFFFF0000u) +
                      tb.z * __uint_as_float(x0.w << 16) + tb.w * __uint_as_float(x0.w & 0xFFFF0000u);
                d1 += ta.x * __uint_as_float(x1.x << 16) + ta.y * __uint_as_float(x1.x & 0xFFFF0000u) +
                      ta.z * __uint_as_float(x1.y << 16) + ta.w * __uint_as_float(x1.y & 0xFFFF0000u) +
                      tb.x * __uint_as_float(x1.z << 16) + tb.y * __uint_as_float(x1.z & 0xFFFF0000u) +
                      tb.z * __uint_as_float(x1.w << 16) + tb.w * __uint_as_float(x1.w & 0xFFFF0000u);
            }
            v.x += d0;
            v.y += d1;
        }
        return v;
    };
    auto store_pair = [&](int row, int cp, float2 v) {
        *reinterpret_cast<__nv_bfloat162 *>(q.C + static_cast<size_t>(m0 + row) * q.n + n0 + 2 * cp) = __floats2bfloat162_rn(v.x, v.y);
    };
    // SwiGLU item `it` of a row: gate pair (it/16)*32 + it%16, up pair 16 further; output columns n0/2 + 2*it, +1
    auto store_item = [&](int row, int it, float2 g, float2 u) {
        const float ox = g.x / (1.f + __expf(-g.x)) * u.x, oy = g.y / (1.f + __expf(-g.y)) * u.y;
        *reinterpret_cast<__nv_bfloat162 *>(q.C + static_cast<size_t>(m0 + row) * (q.n >> 1) + (n0 >> 1) + 2 * it) =
            __floats2bfloat162_rn(ox, oy);
    };
    if (csize == 1) {
        if (!q.swiglu) {
            for (int idx = tid; idx < (m_valid << ppr_shift); idx += nthreads) {
                const int row = idx >> ppr_shift, cp = idx & (ppr - 1);
                store_pair(row, cp, finish_pair(row, cp, team_sum(row, cp)));
            }
        } else {
            for (int idx = tid; idx < (m_valid << (ppr_shift - 1)); idx += nthreads) {
                const int row = idx >> (ppr_shift - 1), it = idx & ((ppr >> 1) - 1);
                const int cg = ((it >> 4) << 5) + (it & 15);
                store_item(row, it, finish_pair(row, cg, team_sum(row, cg)), finish_pair(row, cg + 16, team_sum(row, cg + 16)));
            }
        }
        return;
    }
    const uint32_t recv_base = base + p.off_recv;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    for (int idx = tid; idx < (m_valid << ppr_shift); idx += nthreads) {
        const int row = idx >> ppr_shift, cp = idx & (ppr - 1);
        const float2 v = team_sum(row, cp);
        uint32_t owner, j;
        if (!q.swiglu) {
            owner = __umulhi(static_cast<uint32_t>(cp), p.own_magic);
            j = cp - owner * p.own_cols;
        } else {
            const uint32_t it = static_cast<uint32_t>(((cp >> 5) << 4) + (cp & 15));
            owner = __umulhi(it, p.item_magic);
            j = 2 * (it - owner * p.own_items) + ((cp >> 4) & 1);
        }
        st_async_f2(map_to_cta(recv_base + 8u * ((rank * kRows + row) * p.own_cols + j), owner), v,
                    map_to_cta(base + p.off_mbar, owner));
    }
    // Each CTA goes on as soon as ITS slots are complete (no barrier over the cluster): the stores above count
    // their bytes on the owner's mbarrier.  A CTA that has received everything has nothing left that a peer writes,
    // and its own stores need nothing of it once issued, so it may exit without a second cluster barrier.
    if (!mbar_wait_decode(base + p.off_mbar)) return;
    {
        const float2 *recv = reinterpret_cast<const float2 *>(base_gen + p.off_recv);
        const int slot_stride = kRows * p.own_cols;
        auto rank_sum = [&](int row, int j) {
            const float2 *src = recv + row * p.own_cols + j;
            float2 v = src[0];
#pragma unroll 4
            for (uint32_t r = 1; r < csize; ++r) {
                const float2 u = src[r * slot_stride];
                v.x += u.x;
                v.y += u.y;
            }
            return v;
        };
        if (!q.swiglu) {
            const int cp0 = static_cast<int>(rank) * p.own_cols;
            const int mine = min(p.own_cols, ppr - cp0);  // pairs per row this rank owns (none for a trailing rank)
            for (int idx = tid; idx < m_valid * p.own_cols; idx += nthreads) {
                const int row = static_cast<int>(__umulhi(static_cast<uint32_t>(idx), p.own_magic));
                const int j = idx - row * p.own_cols;
                if (j >= mine) continue;
                store_pair(row, cp0 + j, finish_pair(row, cp0 + j, rank_sum(row, j)));
            }
        } else {
            const int it0 = static_cast<int>(rank) * p.own_items;
            const int mine = min(p.own_items, (ppr >> 1) - it0);
            for (int idx = tid; idx < m_valid * p.own_items; idx += nthreads) {
                const int row = static_cast<int>(__umulhi(static_cast<uint32_t>(idx), p.item_magic));
                const int jj = idx - row * p.own_items;
                if (jj >= mine) continue;
                const int it = it0 + jj, cg = ((it >> 4) << 5) + (it & 15);
                store_item(row, it, finish_pair(row, cg, rank_sum(row, 2 * jj)), finish_pair(row, cg + 16, rank_sum(row, 2 * jj + 1)));
            }
        }
    }
}

// ---- host: decomposition heuristic and launch ---------------------------------------------

struct DecodeConfig {
    int nb, cluster_k, warps_k, warps_n, groups_per_cta, pass_groups;
};

int ceil_div(int a, int b) { return (a + b - 1) / b; }

constexpr int kMaxWarps[3] = {0, KILN_DECODE_LB1 / 32, 16};  // per CTA, by NB (launch bounds of the kernel)
constexpr int kStageBytes = 64 * 1024;     // activations staged per pass

DecodeConfig choose_config(int m, int n, int k, const DecodeOverride &ov) {
    DecodeConfig c{};
    const int groups = k / kGroup, chunks = n / kChunkCols;
    // 9..16 rows per block of CTAs cost two MMAs per packed word and 128 registers; narrow projections (few CTAs, short
    // launches) are faster as several 8-row blocks (k, 2560 -> 512, M=16: 3.8 us against 4.8; M=32: 4.1 against 5.0)
    c.nb = (m <= 8 || (n <= 1024 && m <= 32)) ? 1 : 2;
    const int mblocks = ceil_div(m, 8 * c.nb);
    const int sms = device_sm_count();
    const int warps_sm = c.nb == 1 ? KILN_DECODE_LB1 / 32 : 16;  // resident warps per SM (register file / registers per warp)
    int wn, ck, wk;
    if (ov.cluster_k > 0 && ov.warps_k > 0 && ov.warps_n > 0) {
        ck = ov.cluster_k;
        wk = ov.warps_k;
        wn = ov.warps_n;
    } else {
        // Rule (fitted by eye to sweeps over (cluster_k, warps_k, warps_n) on B200):
        //  * one unit per warp while all warps fit the GPU at once, else as few units per warp as that allows;
        //  * CTAs of half an SM's warps, the K-warps of a 64-column chunk split over as many cluster ranks as that
        //    needs, preferring a cluster size that divides the K groups;
        //  * more than two batch rows: two chunks per CTA (four for wide projections with more than eight rows), so
        //    that the staged activations are shared by more warps;
        //  * a grid far smaller than the GPU is spread over more, smaller CTAs;
        //  * the whole grid must be resident at once (one wave).
        wn = m <= 2 ? 1 : 2;
        if (m > 8 && chunks >= 128) wn = 4;
        while (wn > 1 && chunks % wn) wn /= 2;
        const long long capacity = static_cast<long long>(sms) * warps_sm;
        int kw = groups;  // K-warps per 64-column chunk
        const long long cols = static_cast<long long>(chunks) * mblocks;
        if (cols * kw > capacity) {
            const int fit = static_cast<int>(capacity / cols) > 0 ? static_cast<int>(capacity / cols) : 1;
            kw = ceil_div(groups, ceil_div(groups, fit));
        }
        const int wk_max = (warps_sm / 2) / wn > 0 ? (warps_sm / 2) / wn : 1;
        ck = ceil_div(kw, wk_max);
        if (ck > 8) ck = 8;
        for (int d = ck; d <= 8; ++d)
            if (groups % d == 0) {
                ck = d;
                break;
            }
        if (static_cast<long long>(chunks / wn) * mblocks * ck < sms / 2) ck = groups < 8 ? groups : 8;
        wk = ceil_div(kw, ck);
        if (wk > wk_max) wk = wk_max;
        const long long ctas = static_cast<long long>(chunks / wn) * mblocks * ck;
        while (wk > 1 && ctas > static_cast<long long>(sms) * (warps_sm / (wk * wn))) --wk;
        // Measured exceptions (B200, CUDA-graph replay over rotating weights), keyed by shape and batch class:
        struct Tuned {
            int k, n, m_max, ck, wk, wn;
        };
        static const Tuned kTuned[] = {
            {2560, 4096, 4, 5, 4, 2},    {2560, 4096, 8, 4, 5, 4},   {2560, 4096, 16, 4, 5, 2},   // q
            {2560, 512, 2, 8, 3, 1},     {2560, 512, 4, 5, 4, 2},    {2560, 512, 8, 8, 3, 4},     // k, v
            {2560, 512, 16, 5, 4, 1},
            {4096, 2560, 2, 4, 8, 1},    {4096, 2560, 4, 8, 4, 2},   {4096, 2560, 8, 8, 4, 4},    // o, GDN-out
            {4096, 2560, 16, 6, 6, 2},
            {2560, 18432, 1, 1, 10, 1},  {2560, 18432, 8, 2, 5, 2},  {2560, 18432, 16, 2, 4, 4},  // gate+up
            {9216, 2560, 2, 6, 8, 1},    {9216, 2560, 16, 6, 6, 2},                               // down
            {2560, 8192, 1, 1, 12, 1},   {2560, 8192, 2, 5, 4, 1},   {2560, 8192, 4, 4, 5, 2},    // GDN-in
            {2560, 8192, 8, 4, 5, 4},    {2560, 8192, 16, 4, 4, 4},
        };
        for (const Tuned &t : kTuned)
            if (t.k == k && t.n == n && m <= t.m_max && t.wk * t.wn <= kMaxWarps[c.nb]) {
                ck = t.ck;
                wk = t.wk;
                wn = t.wn;
                break;
            }
    }
    while (wn > 1 && chunks % wn) wn /= 2;
    if (ck > 8) ck = 8;
    if (ck > groups) ck = groups;
    if (ck < 1) ck = 1;
    c.cluster_k = ck;
    c.warps_n = wn;
    c.groups_per_cta = ceil_div(groups, ck);
    if (wk > c.groups_per_cta) wk = c.groups_per_cta;
    if (wk < 1) wk = 1;
    c.warps_k = wk;
    const int rows = m < 8 * c.nb ? m : 8 * c.nb;  // activation rows a CTA stages
    int pg = (kStageBytes / rows - 16) / 256;
    if (pg < 1) pg = 1;
    c.pass_groups = c.groups_per_cta < pg ? c.groups_per_cta : pg;
    return c;
}

template <int NB, bool MULTI>
int launch_list(DecodeParams &p, int ck, int max_m, cudaStream_t stream) {
    static bool attr_set[64] = {};
    constexpr int kMaxSmem = 200 * 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        if (int rc = record_cuda_error(
                cudaFuncSetAttribute(w4a16_decode_kernel<NB, MULTI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem)))
            return rc;
        attr_set[dev] = true;
    }
    // carve-up: [A rows][reduction tiles][receive slots][LoRA: rows of B^T, then scale * x * A^T]
    auto align = [](int x, int a) { return (x + a - 1) / a * a; };
    int a_bytes = 0, lora_bytes = 0, grid_y = 0;
    bool swiglu = false;
    for (int i = 0; i < p.count; ++i) {
        DecodeProblem &q = p.prob[i];
        const int rows = q.m < 8 * NB ? q.m : 8 * NB;
        q.a_pitch = q.pass_groups * 256 + 16;
        a_bytes = std::max(a_bytes, rows * q.a_pitch);
        if (q.lora_r) lora_bytes = std::max(lora_bytes, 64 * p.warps_n * q.lora_r * 2 + 8 * NB * q.lora_r * 4);
        swiglu |= q.swiglu != 0;
        q.y0 = grid_y;
        grid_y += q.n / (kChunkCols * p.warps_n);
    }
    p.red_pitch = p.warps_n * 64 + (NB == 1 ? 4 : 8);  // bank-conflict-free partial stores
    p.off_red = align(a_bytes, 128);
    p.off_recv = p.off_red + align(static_cast<int>(sizeof(float)) * p.warps_k * 8 * NB * p.red_pitch, 128);
    const int ppr = 32 * p.warps_n;  // a power of two: warps_n is 1, 2, 4 or 8
    p.ppr_shift = 5;
    while ((1 << p.ppr_shift) < ppr) ++p.ppr_shift;
    p.own_items = (ppr / 2 + ck - 1) / ck;
    p.own_cols = swiglu ? 2 * p.own_items : (ppr + ck - 1) / ck;
    p.own_magic = static_cast<uint32_t>(((1ull << 32) + p.own_cols - 1) / p.own_cols);
    p.item_magic = static_cast<uint32_t>(((1ull << 32) + p.own_items - 1) / p.own_items);
    p.off_lora = p.off_recv + align(ck > 1 ? 8 * (ck * 8 * NB * p.own_cols) : 0, 128);
    p.off_mbar = p.off_lora + align(lora_bytes, 16);
    const size_t smem = static_cast<size_t>(p.off_mbar) + 16 + 128;
    if (smem > kMaxSmem) return KILN_W4A16_ERR_KERN_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ck, grid_y, (max_m + 8 * NB - 1) / (8 * NB));
    cfg.blockDim = dim3(32 * p.warps_n * p.warps_k);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = ck;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    if (cfg.gridDim.y > 65535 || cfg.gridDim.z > 65535) return KILN_W4A16_ERR_KERN_SHAPE;
    note_launch();
    return record_cuda_error(cudaLaunchKernelEx(&cfg, w4a16_decode_kernel<NB, MULTI>, p));
}

}  // namespace

void decode_plan(int m, int n, int k, const DecodeOverride &ov, int out[4]) {
    const DecodeConfig c = choose_config(m, n, k, ov);
    out[0] = c.cluster_k;
    out[1] = c.warps_k;
    out[2] = c.warps_n;
    out[3] = c.pass_groups;
}

// One launch for `count` independent GEMMs.  The decomposition is the one the rule gives for a single GEMM with the
// tallest m, the longest k and all the columns of the list side by side.
int launch_decode_list(const DecodeItem *items, int count, cudaStream_t stream, const DecodeOverride &ov) {
    if (count < 1 || count > kMaxProblems) return KILN_W4A16_ERR_ARG;
    int max_m = 0, max_k = 0;
    long long sum_n = 0;
    for (int i = 0; i < count; ++i) {
        max_m = std::max(max_m, items[i].m);
        max_k = std::max(max_k, items[i].k);
        sum_n += items[i].n;
    }
    if (sum_n > (1 << 30)) return KILN_W4A16_ERR_KERN_SHAPE;
    const DecodeConfig c = choose_config(max_m, static_cast<int>(sum_n), max_k, ov);
    if (c.warps_n * c.warps_k > kMaxWarps[c.nb] || (c.warps_n & (c.warps_n - 1))) return KILN_W4A16_ERR_KERN_SHAPE;
    DecodeParams p{};
    p.count = count;
    p.warps_n = c.warps_n;
    p.warps_k = c.warps_k;
    for (int i = 0; i < count; ++i) {
        const DecodeItem &it = items[i];
        DecodeProblem &q = p.prob[i];
        if (it.n % (kChunkCols * c.warps_n) != 0) return KILN_W4A16_ERR_KERN_SHAPE;
        if (it.lora_r < 0 || it.lora_r > 128 || it.lora_r % 8 != 0) return KILN_W4A16_ERR_ARG;
        q.A = static_cast<const __nv_bfloat16 *>(it.A);
        q.B = static_cast<const uint4 *>(it.B);
        q.S = static_cast<const __half *>(it.S);
        q.C = static_cast<__nv_bfloat16 *>(it.C);
        q.lora_t = it.lora_r ? static_cast<const float *>(it.lora_t) : nullptr;
        q.lora_b = static_cast<const __nv_bfloat16 *>(it.lora_b);
        q.lora_r = it.lora_r;
        q.swiglu = it.swiglu;
        q.m = it.m;
        q.n = it.n;
        q.k = it.k;
        q.groups = it.k / kGroup;
        q.groups_per_cta = ceil_div(q.groups, c.cluster_k);
        const int rows = it.m < 8 * c.nb ? it.m : 8 * c.nb;
        int pg = (kStageBytes / rows - 16) / 256;
        if (pg < 1) pg = 1;
        q.pass_groups = q.groups_per_cta < pg ? q.groups_per_cta : pg;
        q.per_column = it.groupsize == -1;
    }
    if (c.nb == 1)
        return count == 1 ? launch_list<1, false>(p, c.cluster_k, max_m, stream) : launch_list<1, true>(p, c.cluster_k, max_m, stream);
    return count == 1 ? launch_list<2, false>(p, c.cluster_k, max_m, stream) : launch_list<2, true>(p, c.cluster_k, max_m, stream);
}

int launch_decode(const GemmArgs &a, const DecodeOverride &ov) {
    DecodeItem it{};
    it.A = a.A;
    it.B = a.B;
    it.S = a.S;
    it.C = a.C;
    it.m = a.m;
    it.n = a.n;
    it.k = a.k;
    it.groupsize = a.groupsize;
    it.lora_t = a.lora_t;
    it.lora_b = a.lora_b;
    it.lora_r = a.lora_r;
    it.swiglu = a.swiglu;
    return launch_decode_list(&it, 1, a.stream, ov);
}

// Reads and clears this device's decode status word (set when a CTA gave up waiting for its cluster peers).
int decode_status_read_clear(cudaStream_t st, uint32_t *out) {
    *out = 0;
    void *w = nullptr;
    if (int rc = record_cuda_error(cudaGetSymbolAddress(&w, g_decode_status))) return rc;
    if (int rc = record_cuda_error(cudaMemcpyAsync(out, w, sizeof(uint32_t), cudaMemcpyDeviceToHost, st))) return rc;
    if (int rc = record_cuda_error(cudaStreamSynchronize(st))) return rc;
    if (*out != 0) {
        if (int rc = record_cuda_error(cudaMemsetAsync(w, 0, sizeof(uint32_t), st))) return rc;
        if (int rc = record_cuda_error(cudaStreamSynchronize(st))) return rc;
    }
    return 0;
}

}  // namespace kiln
