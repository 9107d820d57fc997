// W4A16 GEMM for 17..128 activation rows on sm_100a: the dequantised weights are the TENSOR-MEMORY operand of tcgen05.mma.
//
// The general tcgen05 kernel (prefill_w4a16_umma.cu) dequantises a 128-column weight tile into shared memory, where the
// MMA reads it back together with a 128-row activation tile.  For a problem with few rows that costs, per 128 K, 32 KB of
// weights and 32 KB of activations written to shared memory and 64 KB read by the MMAs, four 4-byte shared-memory stores
// per packed word on top of the dequant arithmetic, and MMAs of 128 rows whatever the number of real ones (measured:
// gate+up 2560 -> 18432 takes 16.4 us from M=33 to M=128, 0.55 us per 128 K, with every role idle half of the time).
// Here the GEMM is issued transposed, C^T[n, m] = W^T[n, k] * X^T[k, m]:
//  * the 128 weight columns of a tile are the M = 128 rows of the MMA, one per TMEM lane, and the dequant warps write
//    them straight into tensor memory with tcgen05.st (bf16 pairs of consecutive K per 32-bit cell); they never
//    touch shared memory;
//  * the activations are the N operand (N = rows rounded up to 16, at most 128), K-major 128B-swizzled tiles that TMA
//    drops into shared memory: at most 32 KB per 128 K, written once and read once;
//  * the accumulator is 128 lanes x N fp32 columns; a thread of the epilogue owns one output column.
// A packed word of the kiln-marlin-gemm layout (kiln-marlin-gemm/src/lib.rs:262-357) gives a lane two K pairs of eight
// columns, but a TMEM lane needs all K of ONE column: the four lanes of a quad exchange their PACKED bytes (two
// shuffles and a few byte permutes per 16 K, a quarter of the data of a transpose after dequantisation), after which
// lane (c, qd) of the warp that owns TMEM lanes 32x..32x+31 holds column 64*(x/2) + 16*(2*(x%2) + qd/2) + 8*(qd%2) + c
// of the tile.  That lane <-> column permutation is undone by the epilogue's store addresses.
// Roles (480 threads): warp 0 TMA producer, warps 1 and 14 MMA issuers (each issues four of the eight K=16 MMAs of a
// stage into an accumulator of its own: one thread issues about one tcgen05.mma per 105 cycles), warps 2-5 epilogue,
// warps 6-13 dequant in two teams of four warps (a team covers the four lane quarters) that take the stages in turn.
// The K loop is bound by the dequant instruction stream on the integer pipe (about 40 instructions per 16 K and lane).
// SwiGLU (gate and up columns interleaved in runs of 32, no K split): the warp that owns a run of gate columns and the warp
// that owns their up columns put their sums into shared memory and each writes silu(gate) * up for half of the rows.
// LoRA delta (grouped scales): one extra stage at the start of a tile's K range, its tensor-memory operand the tile's rows of
// lora_b and its activation tile t = scale * x * A^T (bf16, written by the kernel launched just before).
// Every wait is bounded (w4a16_async.cuh); K splits write fp32 slabs that splitk_reduce_kernel sums.  Per-column scales
// (group size -1): the weights are dequantised unscaled and the scale multiplies the finished sums.
#include "w4a16_common.cuh"
#include "w4a16_umma.cuh"

namespace kiln {
namespace {

constexpr int kTileCols = 128;                   // weight columns per tile = TMEM lanes = MMA M
constexpr int kMaxRows = 128;                    // most activation rows = MMA N (rounded up to 16) the kernel takes
constexpr int kStageK = 128;                     // K per pipeline stage: one scale group, eight K=16 MMAs
constexpr int kStages = 4;
// The kernel comes in two sizes, R = 64 or 128 rows: an activation atom is R rows x 64 bf16 (128B-swizzled), a stage
// two atoms, an accumulator R fp32 columns.  R = 64 has two accumulator buffers per issuer (a CTA with several units
// drains one while the next fills), R = 128 one: 4 x 64 + 2 x 2 x 64 = 4 x 64 + 2 x 128 = 512 TMEM columns either way.
constexpr int kWStageCols = kStageK / 2;         // TMEM columns of one stage of weights (two bf16 per cell)
constexpr int kAccBase = kStages * kWStageCols;  // accumulators start at TMEM column 256
constexpr int kTmemCols = 512;                   // 256 of weights + 256 of accumulators
constexpr int kDequantWarp0 = 6, kTeamWarps = 4, kTeams = 2;
constexpr int kIssuerWarp2 = kDequantWarp0 + kTeamWarps * kTeams;
constexpr int kThreads = (kIssuerWarp2 + 1) * 32;
constexpr int kBarrierBytes = 256;
template <int R, bool SWIGLU>
constexpr int smem_bytes() {  // stages, barriers, the SwiGLU exchange area (two warp pairs x gate and up x R rows x 32 floats), alignment slack
    return kStages * 2 * R * 128 + kBarrierBytes + (SWIGLU ? 4 * R * 32 * 4 : 0) + 1024;
}

struct SmallMParams {
    const uint2 *B;  // packed weights seen as 8-byte halves of the 16-byte lane pieces
    const __half *S;
    __nv_bfloat16 *C;
    float *partial;  // fp32 [splits][m][n] when splits > 1
    uint32_t *status;
    int m, n, n_tiles, splits, k_stages, npad;
    // LoRA delta C += t * lora_b^T: t = scale * x * A^T is bf16 [m, lora_r] (its tensor map is the kernel's second), lora_b
    // bf16 [n, lora_r], lora_r a multiple of 8 up to 128.  The unit that starts a tile's K range begins with one extra
    // stage whose tensor-memory operand is the tile's rows of lora_b and whose activation tile is t.
    const __nv_bfloat16 *lora_b;
    int lora_r;
    int swiglu;      // columns hold gate and up interleaved in runs of 32; C is [m, n/2] = silu(gate) * up (splits == 1 only)
    int per_column;  // one fp16 scale per column (group size -1): dequantised unscaled, the scale applied to the sums
    unsigned long long wait_limit_ns;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint2 ld_stream_v2(const uint2 *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const __half *p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
                 "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
// named barrier of the two epilogue warps that share a 64-column chunk (ids 1 and 2; 0 is __syncthreads)
__device__ __forceinline__ void pair_barrier(int ch) {
    if (ch == 0)
        asm volatile("bar.sync 1, 64;" ::: "memory");
    else
        asm volatile("bar.sync 2, 64;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A = 128 lanes x 8 cells (16 K as bf16 pairs), B = K-major tile of N rows
__device__ __forceinline__ void umma_bf16_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// SWIGLU is a template parameter so that the plain kernel's epilogue is compiled on its own (with the option as a run-time
// branch the plain epilogue came out 6-27 % slower for 64-128 rows).
template <int R, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
w4a16_smallm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_t, const SmallMParams p) {
    constexpr int kXAtomBytes = R * 128, kXStageBytes = 2 * kXAtomBytes;
    constexpr int kAccBufs = R == 64 ? 2 : 1;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kStages * kXStageBytes;
    auto full = [&](int s) { return bar_base + 8u * s; };                       // TMA bytes + the arrivals of one dequant team
    auto empty = [&](int s) { return bar_base + 8u * (kStages + s); };          // one tcgen05.commit per issuer
    auto tmem_full = [&](int a) { return bar_base + 8u * (2 * kStages + a); };  // one commit per issuer
    auto tmem_empty = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    uint8_t *bar_gen = smem_gen + kStages * kXStageBytes;
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bar_gen + 8 * (2 * kStages + 4));
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bar_gen + 8 * (2 * kStages + 4) + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full(s), 1 + kTeamWarps * 32);
            mbar_init(empty(s), 2);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full(a), 2);
            mbar_init(tmem_empty(a), 128);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t *>(tmem_ptr_slot))),
                     "r"(static_cast<uint32_t>(kTmemCols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp == 0 && lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_slot;
    // The packed weights and scales never depend on the previous kernel in the stream: only the roles that read the
    // activations or write C order themselves after it.
    pdl_launch_dependents();

    const int units = p.n_tiles * p.splits;
    // unit u = (tile u / splits, split u % splits); a split covers the stages [sp * k_stages / splits, (sp+1) * ...)
    auto unit_range = [&](int u, int &nt, int &sp, int &ks0, int &ks1) {
        nt = u / p.splits;
        sp = u - nt * p.splits;
        ks0 = sp * p.k_stages / p.splits;
        ks1 = (sp + 1) * p.k_stages / p.splits;
    };
    int nt, sp, ks0, ks1;
    // stage "ks0 - 1" of a unit with sp == 0 is the LoRA stage, when there is a delta
    auto lora_pre = [&](int sp_) { return (p.lora_r > 0 && sp_ == 0) ? 1 : 0; };

    if (warp == 0) {
        // ---------------- TMA producer: activations ----------------
        if (lane == 0) {
            pdl_wait();  // the activations may be the previous kernel's output
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                unit_range(u, nt, sp, ks0, ks1);
                for (int ks = ks0 - lora_pre(sp); ks < ks1; ++ks, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, 0xA00u | s, p.wait_limit_ns))) break;
                    mbar_arrive_expect_tx(full(s), static_cast<uint32_t>(p.npad) * 256u);  // (rows past m are zero-filled and counted)
                    const CUtensorMap *map = ks < ks0 ? &tmap_t : &tmap_x;  // (columns of t past lora_r read zero)
                    const int x0 = ks < ks0 ? 0 : ks * kStageK;
                    tma_load_2d(smem_base + s * kXStageBytes, map, x0, 0, full(s));
                    tma_load_2d(smem_base + s * kXStageBytes + kXAtomBytes, map, x0 + 64, 0, full(s));
                }
            }
            if (!ok) {  // drain: wait (bounded, ignoring the abort flag) for copies already issued
                const uint32_t first = it >= static_cast<uint32_t>(kStages) ? it - kStages : 0;
                for (uint32_t j = first; j < it; ++j) mbar_wait_quiet(full(j % kStages), (j / kStages) & 1);
            }
        }
    } else if (warp == 1 || warp == kIssuerWarp2) {
        // ---------------- MMA issuers ----------------
        if (lane == 0) {
            const int q = warp == 1 ? 0 : 1;  // MMAs 4q .. 4q+3 of every stage, accumulator q
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(p.npad >> 3) << 17) |
                                   (static_cast<uint32_t>(kTileCols >> 4) << 24);  // D fp32, A/B bf16, K-major, N = npad, M = 128
            uint32_t it = 0, tile = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++tile) {
                unit_range(u, nt, sp, ks0, ks1);
                const uint32_t acc = tile % kAccBufs, acc_ph = (tile / kAccBufs) & 1;
                const uint32_t d_tmem = tmem_base + kAccBase + (acc * 2 + q) * R;
                const int ksf = ks0 - lora_pre(sp);  // first stage of the unit
                for (int ks = ksf; ks < ks1; ++ks, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!(ok = mbar_wait(full(s), ph, abort_flag, p.status, 0xB00u | s, p.wait_limit_ns))) break;
                    if (ks == ksf) {  // first write into this accumulator: the epilogue must have drained it
                        if (!(ok = mbar_wait(tmem_empty(acc), acc_ph ^ 1, abort_flag, p.status, 0xC00u | acc, p.wait_limit_ns))) break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int kg = 4 * q + j;  // K=16 slice of the stage: atom q, slice j
                        const uint64_t b_desc = make_smem_desc(smem_base + s * kXStageBytes + q * kXAtomBytes) + 2 * j;
                        umma_bf16_tmem_a(d_tmem, tmem_base + s * kWStageCols + kg * 8, b_desc, idesc, (ks > ksf || j > 0) ? 1u : 0u);
                    }
                    umma_commit(empty(s));
                    if (ks == ks1 - 1) umma_commit(tmem_full(acc));
                }
            }
        }
    } else if (warp < kDequantWarp0) {
        // ---------------- epilogue: a thread owns one output column, all rows ----------------
        const int quarter = warp & 3, c = lane >> 2, qd = lane & 3;
        const int col_in_tile = 64 * (quarter >> 1) + 16 * (2 * (quarter & 1) + (qd >> 1)) + 8 * (qd & 1) + c;
        pdl_wait();  // C (or the workspace) may still be read or written by the previous kernel
        uint32_t tile = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x, ++tile) {
            unit_range(u, nt, sp, ks0, ks1);
            const uint32_t acc = tile % kAccBufs, acc_ph = (tile / kAccBufs) & 1;
            if (!(ok = mbar_wait(tmem_full(acc), acc_ph, abort_flag, p.status, 0xD00u | acc, p.wait_limit_ns))) break;
            tc_fence_after();
            const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kAccBase + acc * 2 * R;
            const size_t col = static_cast<size_t>(nt) * kTileCols + col_in_tile;
            // per-column scales: applied here when the tile is complete, by the split-K reduction otherwise
            const float cs = (p.per_column && p.splits == 1) ? __half2float(p.S[scale_single_pos(static_cast<int>(col))]) : 1.f;
            if constexpr (SWIGLU) {
                // A 64-column chunk is a run of 32 gate columns and the 32 up columns that go with them: this warp owns
                // one run, the warp of the neighbouring lane quarter the other, column for column in the same lanes.
                // Both put their sums into shared memory, then each computes silu(gate) * up for half of the rows.
                const int hf = quarter & 1, ch = quarter >> 1;
                float *xg = reinterpret_cast<float *>(bar_gen + kBarrierBytes) + ch * (2 * R * 32), *xu = xg + R * 32;
                float *mine = hf ? xu : xg;
                for (int r0 = 0; r0 < p.npad; r0 += 16) {
                    uint32_t a[16], b[16];
                    tmem_ld_32x32b_x16(t0 + r0, a);
                    tmem_ld_32x32b_x16(t0 + R + r0, b);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) mine[(r0 + i) * 32 + lane] = (__uint_as_float(a[i]) + __uint_as_float(b[i])) * cs;
                }
                // (both warps of a pair come here after the same mbarrier wait above, and leave together)
                pair_barrier(ch);
                // (a lane holds the same column of its run in both warps: col_in_tile % 32)
                const size_t ocol = static_cast<size_t>(nt) * (kTileCols / 2) + ch * 32 + (col_in_tile & 31);
                const int half = p.npad >> 1, r_end = min(p.m, (hf + 1) * half);
#pragma unroll 4
                for (int r = hf * half; r < r_end; ++r) {
                    const float g = xg[r * 32 + lane], u = xu[r * 32 + lane];
                    p.C[static_cast<size_t>(r) * (p.n >> 1) + ocol] = __float2bfloat16_rn(__fdividef(g, 1.f + __expf(-g)) * u);
                }
                pair_barrier(ch);  // the exchange area may be written again
            } else
            for (int r0 = 0; r0 < p.npad; r0 += 16) {
                uint32_t a[16], b[16];
                tmem_ld_32x32b_x16(t0 + r0, a);
                tmem_ld_32x32b_x16(t0 + R + r0, b);
                tmem_ld_wait();
                if (p.splits == 1) {
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (r0 + i < p.m)
                            p.C[static_cast<size_t>(r0 + i) * p.n + col] =
                                __float2bfloat16_rn((__uint_as_float(a[i]) + __uint_as_float(b[i])) * cs);
                } else {
                    float *dst = p.partial + static_cast<size_t>(sp) * p.m * p.n + col;
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (r0 + i < p.m) dst[static_cast<size_t>(r0 + i) * p.n] = __uint_as_float(a[i]) + __uint_as_float(b[i]);
                }
            }
            tc_fence_before();
            mbar_arrive(tmem_empty(acc));
        }
    } else if (warp < kIssuerWarp2) {
        // ---------------- dequant: packed int4 -> bf16 pairs in tensor memory ----------------
        const int team = (warp - kDequantWarp0) / kTeamWarps;  // warps 6-9 / 10-13: each team has one warp per lane quarter
        const int quarter = warp & 3, ch = quarter >> 1, hf = quarter & 1;
        const int c = lane >> 2, qd = lane & 3;
        const int chunks_n = p.n >> 6;
        // Byte-permute selectors of the quad exchange (see the loop).  Bytes of a packed word: 0 = column 16j+c, even K;
        // 1 = column 16j+8+c, even K; 2, 3 = the same columns, odd K; in each byte the low nibble is K pair qd, the high
        // nibble K pair qd+4.  "Item" i = {even byte, odd byte} of the lane's column i = 2*(j - 2hf) + e: bytes (0,2) and
        // (1,3) of the lane's first word, (4,6) and (5,7) of its second.
        const uint32_t selK = (qd & 1) ? 0x7531u : 0x6420u;  // the two items this lane keeps in the exchange with lane qd^1 ...
        const uint32_t selS = (qd & 1) ? 0x6420u : 0x7531u;  // ... and the two it sends
        // after it, {kept, received} hold items {b0, 2+b0} (b0 = qd%2) of the lane pair's two source lanes; ordered by source:
        const uint32_t selU = (qd & 1) ? 0x1054u : 0x5410u, selV = (qd & 1) ? 0x3276u : 0x7632u;  // item b0 / item 2+b0
        const uint32_t selK2 = (qd & 2) ? selV : selU;       // exchange with lane qd^2: keep the item this lane owns (item qd) ...
        const uint32_t selS2 = (qd & 2) ? selU : selV;       // ... send the other
        const uint32_t selRa = (qd & 2) ? 0x7564u : 0x3120u, selRb = (qd & 2) ? 0x3120u : 0x7564u;
        // this lane's column after the exchange is 16 * (2hf + qd/2) + 8 * (qd%2) + c of chunk ch; its scale sits at
        // 8c + 2hf*2 + qd of the chunk's scale order (position 8i + t holds column 8t + i)
        const int scale_off = ch * 64 + 8 * c + 4 * hf + qd;
        const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        uint32_t it_base = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
            unit_range(u, nt, sp, ks0, ks1);
            const uint2 *wbase = p.B + (static_cast<size_t>(nt * 2 + ch) * 32 + lane) * 2 + hf;
            const __half *sbase = p.S + static_cast<size_t>(nt) * kTileCols + scale_off;
            auto load_stage = [&](uint2 (&d)[8], uint32_t &sc, int ks) {
#pragma unroll
                for (int kt = 0; kt < 8; ++kt) d[kt] = ld_stream_v2(wbase + static_cast<size_t>(ks * 8 + kt) * chunks_n * 64);
                sc = p.per_column ? 0x3C00u : ld_stream_u16(sbase + static_cast<size_t>(ks) * p.n);  // (fp16 1.0)
            };
            if (lora_pre(sp)) {
                // LoRA stage: the tensor-memory operand is this tile's rows of lora_b, one row per lane, K = lora_r padded
                // with zeros to 128.  A weight like any other: it is read without waiting for the previous kernel.
                if (it_base % kTeams == static_cast<uint32_t>(team)) {
                    const int s = it_base % kStages;
                    const uint32_t ph = (it_base / kStages) & 1;
                    const int col_in_tile = 64 * ch + 16 * (2 * hf + (qd >> 1)) + 8 * (qd & 1) + c;
                    const uint4 *row = reinterpret_cast<const uint4 *>(p.lora_b + (static_cast<size_t>(nt) * kTileCols + col_in_tile) * p.lora_r);
                    if ((ok = mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, 0xE00u | s, p.wait_limit_ns))) {
                        tc_fence_after();
#pragma unroll 1
                        for (int h = 0; h < 4; ++h) {  // four K tiles of 16 = four pairs of 16-byte pieces at a time (few registers)
                            uint4 lw[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                lw[i] = 8 * (4 * h + i) + 8 <= p.lora_r ? ld_stream_v4(row + 4 * h + i) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                            for (int kt = 0; kt < 2; ++kt) {
                                const uint32_t r[8] = {lw[2 * kt].x, lw[2 * kt].y, lw[2 * kt].z, lw[2 * kt].w,
                                                       lw[2 * kt + 1].x, lw[2 * kt + 1].y, lw[2 * kt + 1].z, lw[2 * kt + 1].w};
                                tmem_st_32x32b_x8(t_lane + s * kWStageCols + (2 * h + kt) * 8, r);
                            }
                        }
                        tmem_st_wait();
                        tc_fence_before();
                        mbar_arrive(full(s));
                    }
                }
                ++it_base;
                if (!ok) break;
            }
            // this team's stages of the unit: those whose running stage number is congruent to `team`
            const int kf = ks0 + static_cast<int>((static_cast<uint32_t>(team) + kTeams - it_base % kTeams) % kTeams);
            // Packed words and scales of the team's next three stages are always in flight, each stage's in registers of
            // its own (the loop is unrolled three times so that no register with a pending load is ever copied).
            uint2 rw[3][8];
            uint32_t rs[3];
#pragma unroll
            for (int v = 0; v < 3; ++v) {
                rs[v] = 0;
                if (kf + v * kTeams < ks1) load_stage(rw[v], rs[v], kf + v * kTeams);
            }
            for (int kb = kf; kb < ks1 && ok; kb += 3 * kTeams) {
#pragma unroll
                for (int v = 0; v < 3; ++v) {
                    const int ks = kb + v * kTeams;
                    if (ks >= ks1) break;
                    const uint32_t it = it_base + static_cast<uint32_t>(ks - ks0);
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    __nv_bfloat162 scale2;
                    {
                        const float f = __half2float(__ushort_as_half(static_cast<unsigned short>(rs[v])));
                        scale2 = __floats2bfloat162_rn(f, f);
                    }
                    if (!(ok = mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, 0xE00u | s, p.wait_limit_ns))) break;
                    tc_fence_after();
#pragma unroll
                    for (int kt = 0; kt < 8; ++kt) {
                        // 4 x 4 transpose of the 16-bit items over the quad, on the packed bytes: lane qd ends up with item qd
                        // (its column) of lanes 0..3, i.e. all eight K pairs of the 16-row K tile
                        const uint32_t keep1 = prmt(rw[v][kt].x, rw[v][kt].y, selK);
                        const uint32_t recv1 = __shfl_xor_sync(0xFFFFFFFFu, prmt(rw[v][kt].x, rw[v][kt].y, selS), 1);
                        const uint32_t keep2 = prmt(keep1, recv1, selK2);
                        const uint32_t recv2 = __shfl_xor_sync(0xFFFFFFFFu, prmt(keep1, recv1, selS2), 2);
                        // ra: even-K nibbles of K pairs 0, 4, 1, 5 in bits 0..15, the odd-K ones in bits 16..31; rb: pairs 2, 6, 3, 7
                        const uint32_t ra = prmt(keep2, recv2, selRa), rb = prmt(keep2, recv2, selRb);
                        uint32_t r[8];
                        r[0] = lop3_and_or(ra, kNibMask, kMagic128);
                        r[4] = lop3_and_or(ra >> 4, kNibMask, kMagic128);
                        r[1] = lop3_and_or(ra >> 8, kNibMask, kMagic128);
                        r[5] = lop3_and_or(ra >> 12, kNibMask, kMagic128);
                        r[2] = lop3_and_or(rb, kNibMask, kMagic128);
                        r[6] = lop3_and_or(rb >> 4, kNibMask, kMagic128);
                        r[3] = lop3_and_or(rb >> 8, kNibMask, kMagic128);
                        r[7] = lop3_and_or(rb >> 12, kNibMask, kMagic128);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {  // (128 + nibble) - 136, times the group scale: the same two roundings as the general kernel
                            __nv_bfloat162 w = *reinterpret_cast<__nv_bfloat162 *>(&r[e]);
                            const uint32_t k136 = kPos136x2;
                            w = __hsub2(w, *reinterpret_cast<const __nv_bfloat162 *>(&k136));
                            w = __hmul2(w, scale2);
                            r[e] = *reinterpret_cast<uint32_t *>(&w);
                        }
                        tmem_st_32x32b_x8(t_lane + s * kWStageCols + kt * 8, r);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                    mbar_arrive(full(s));
                    if (ks + 3 * kTeams < ks1) load_stage(rw[v], rs[v], ks + 3 * kTeams);
                }
            }
            it_base += static_cast<uint32_t>(ks1 - ks0);
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(static_cast<uint32_t>(kTmemCols))
                     : "memory");
    }
}

}  // namespace

// Shapes this kernel takes (any row count up to 128 works; the dispatcher decides from which one it pays).
bool smallm_supported(int m, int n, int k, int groupsize) {
    return m >= 1 && m <= kMaxRows && (groupsize == 128 || groupsize == -1) && n % kTileCols == 0 && k % kStageK == 0;
}

// C = A * dequant(B) with `splits` K splits (fp32 slabs of m * n in `partial` when splits > 1, summed by the caller).
int launch_smallm(const GemmArgs &a, int splits, float *partial) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return KILN_W4A16_ERR_CUDA;
    uint32_t *status = device_status_word();
    if (!status) return KILN_W4A16_ERR_CUDA;
    if (splits < 1 || splits > a.k / kStageK || (splits > 1 && !partial) || (a.swiglu && splits != 1)) return KILN_W4A16_ERR_KERN_SHAPE;

    CUtensorMap tmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k) * 2};
    const int npad = (a.m + 15) & ~15;
    const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(npad)};  // (the MMA reads npad rows of the 64-row slots)
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.A), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return KILN_W4A16_ERR_CUDA;

    CUtensorMap tmap_t = tmap;  // (unused without a LoRA delta)
    const bool lora = a.lora_r > 0 && a.lora_t && a.lora_b;
    if (lora) {
        if (a.groupsize == -1 || a.lora_r % 8 != 0 || a.lora_r > 128) return KILN_W4A16_ERR_KERN_SHAPE;
        const cuuint64_t td[2] = {static_cast<cuuint64_t>(a.lora_r), static_cast<cuuint64_t>(a.m)};
        const cuuint64_t ts[1] = {static_cast<cuuint64_t>(a.lora_r) * 2};
        if (enc(&tmap_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.lora_t), td, ts, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return KILN_W4A16_ERR_CUDA;
    }

    SmallMParams p{};
    p.B = static_cast<const uint2 *>(a.B);
    p.S = static_cast<const __half *>(a.S);
    p.C = static_cast<__nv_bfloat16 *>(a.C);
    p.partial = partial;
    p.status = status;
    p.m = a.m;
    p.n = a.n;
    p.n_tiles = a.n / kTileCols;
    p.splits = splits;
    p.k_stages = a.k / kStageK;
    p.npad = npad;
    p.per_column = a.groupsize == -1;
    p.swiglu = a.swiglu;
    p.lora_b = lora ? static_cast<const __nv_bfloat16 *>(a.lora_b) : nullptr;
    p.lora_r = lora ? a.lora_r : 0;
    p.wait_limit_ns = current_wait_limit_ns();

    static bool attr_set[4][64] = {};  // per kernel variant and device: the shared-memory attribute is set once
    int dev = 0;
    cudaGetDevice(&dev);
    auto launch = [&](auto kernel, int smem, int variant) -> int {
        if (dev < 64 && !attr_set[variant][dev]) {
            if (int rc = record_cuda_error(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem))) return rc;
            attr_set[variant][dev] = true;
        }
        const int units = p.n_tiles * p.splits;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(units < device_sm_count() ? units : device_sm_count());
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = a.stream;
        cudaLaunchAttribute attr = pdl_attribute();
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        note_launch();
        return record_cuda_error(cudaLaunchKernelEx(&cfg, kernel, tmap, tmap_t, p));
    };
    if (a.swiglu)
        return a.m <= 64 ? launch(w4a16_smallm_kernel<64, true>, smem_bytes<64, true>(), 2)
                         : launch(w4a16_smallm_kernel<128, true>, smem_bytes<128, true>(), 3);
    return a.m <= 64 ? launch(w4a16_smallm_kernel<64, false>, smem_bytes<64, false>(), 0)
                     : launch(w4a16_smallm_kernel<128, false>, smem_bytes<128, false>(), 1);
}

}  // namespace kiln
