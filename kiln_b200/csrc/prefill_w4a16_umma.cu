// Prefill-shape W4A16 GEMM for sm_100a: TMA-fed tcgen05 (UMMA) GEMM with TMEM accumulators
// and the int4 -> bf16 dequant fused into the shared-memory staging of the B operand.
//
// Replaces the reference's `Marlin<256,{1..4},16,4,4,8>` path
// (kiln-marlin-gemm/csrc/marlin_kernel.cu:197-700, dispatch :784-816: 64-row m-tiles,
// mma.sync, host loop over M) with a persistent, warp-specialised kernel:
//
//   warp 0      TMA producer: activation tiles A[128 x 64] bf16 -> 128B-swizzled smem
//   warp 1      MMA issuer: tcgen05.mma 128 x BN x 16, fp32 accumulators in TMEM (two buffers);
//               also owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld TMEM -> registers -> bf16 -> global (or fp32 split-K slabs)
//   warps 6-13  dequant: packed int4 words (16 B per lane, straight from global/L2) ->
//               bf16 (nib-8)*scale -> the K-major 128B-swizzled B tile the MMA reads
//
// The Marlin fragment layout maps onto the swizzled K-major tile with conflict-free 4-byte
// stores: lane (qd, c) owns K-pairs (2qd, 2qd+1), (2qd+8, 2qd+9) of column 8t + c, and the
// 128B swizzle XORs the 16-byte chunk index with (column % 8) = c.
//
// Every wait in the kernel is bounded: a wait that runs out records an error code in the
// device status word, raises a CTA-wide abort flag that every other wait polls, and the CTA
// drains its outstanding TMA copies, frees its TMEM and returns.
#include <mutex>

#include "w4a16_umma.cuh"

namespace kiln {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kDequantWarp0 = 6;
constexpr uint32_t kEpiWarpBytes = 4096;  // per epilogue warp: 32 rows x 64 columns of bf16, 128B-swizzled (four 1024-byte atoms)
constexpr int kNumEpilogueThreads = 4 * 32;

struct PrefillParams {
    const uint4 *B;
    const __half *S;
    __nv_bfloat16 *C;
    float *partial;  // fp32 [splits][m][n] when splits > 1
    uint32_t *status;
    int m, n, k;
    int m_tiles, n_tiles, splits, k_iters;  // k_iters = k / 64
    int per_column;
    // fused all-gather epilogue: n_peers > 0 -> every finished tile row segment is stored to the row-major
    // [m, ldc] buffer of each peer GPU (peer_c[i], plain peer-mapped pointers) at column offset col0
    __nv_bfloat16 *peer_c[8];
    int n_peers, ldc, col0;
    int self_peer;  // index in peer_c of the buffer that lives on this GPU (written through the TMA store), or -1
    int swiglu;     // columns hold gate and up interleaved in runs of 32; C is [m, n/2] = silu(gate) * up (whole tiles, KP == 1)
    // LoRA delta as extra K-steps: the piece of work that starts a tile's K range appends lora_steps (1 or 2) 64-deep steps
    // whose operands are bf16 tiles of t = scale * x * A^T [m, r] and of lora_b [n, r], both fetched by TMA (KS == 1 only)
    int lora_steps;
    // mc_c != nullptr: one multimem.st per piece to the group's multicast address instead (the switch replicates
    // the store into every GPU's buffer, this GPU's included, so each tile leaves this GPU once)
    __nv_bfloat16 *mc_c;
    int stream_k;     // 1: whole waves of tiles round-robin, then the remaining tiles' (tile, K-step) space in equal shares
    int sk_first_tile;  // stream-K: tiles below this index are dealt whole (a multiple of the grid size)
    int sk_ctas;        // stream-K: CTAs that share the remaining tiles (<= grid size)
    int tile_elems;   // rows * columns of one output tile (stream-K slabs are tile-shaped)
    unsigned long long wait_limit_ns;  // every bounded wait of the launch gives up after this long
    int test_drop_a_load;  // test hook: the activation tile of this K-step (counted per CTA) is announced but never copied; -1 = off
};

// Hands a CTA its work.  Default: units (tile, K-split) dealt round-robin.  Stream-K (hybrid): the tiles that fill
// whole waves of the grid are dealt round-robin as above; the flattened (tile, K-step) space of the remaining
// tiles is cut into sk_ctas equal contiguous ranges, so no SM idles in a last partial wave; a range covers the
// tail of one tile, whole tiles, and the head of another.  Whole tiles are written straight to C; the at most
// two partial pieces of a CTA go to fp32 slabs 2*cta and 2*cta+1 of the workspace and are summed per tile, in
// CTA order, by `streamk_fixup_kernel`.  No CTA waits for another.
struct WorkIter {
    int mode, u, units, stride, splits, m_tiles, k_iters, first_tile;
    long long cur, begin, end;
    __device__ WorkIter(const PrefillParams &p)
        : mode(p.stream_k), u(blockIdx.x), units(p.m_tiles * p.n_tiles * p.splits), stride(gridDim.x), splits(p.splits),
          m_tiles(p.m_tiles), k_iters(p.k_iters), first_tile(p.sk_first_tile) {
        if (mode) {
            units = first_tile;  // whole tiles of the full waves (splits == 1 in this mode)
            const long long total = static_cast<long long>(p.m_tiles * p.n_tiles - first_tile) * p.k_iters;
            const long long c = blockIdx.x, n = p.sk_ctas;
            begin = cur = c < n ? total * c / n : 0;
            end = c < n ? total * (c + 1) / n : 0;
        } else {
            begin = cur = end = 0;
        }
    }
    // slab: -1 = the piece is a whole tile (or an ordinary split) and goes where `sp` says; >= 0 = stream-K slab index
    __device__ bool next(int &mt, int &nt, int &sp, int &ki0, int &ki1, int &slab) {
        if (u < units) {
            sp = u % splits;
            const int t = u / splits;
            mt = t % m_tiles;
            nt = t / m_tiles;
            ki0 = static_cast<int>(static_cast<long long>(k_iters) * sp / splits);
            ki1 = static_cast<int>(static_cast<long long>(k_iters) * (sp + 1) / splits);
            slab = -1;
            u += stride;
            return true;
        }
        if (cur >= end) return false;
        const int tr = static_cast<int>(cur / k_iters);  // tile within the remainder
        ki0 = static_cast<int>(cur - static_cast<long long>(tr) * k_iters);
        const long long left = end - cur;
        ki1 = left < k_iters - ki0 ? ki0 + static_cast<int>(left) : k_iters;
        const int t = first_tile + tr;
        mt = t % m_tiles;
        nt = t / m_tiles;
        sp = 0;
        slab = (ki0 == 0 && ki1 == k_iters) ? -1 : 2 * static_cast<int>(blockIdx.x) + (cur == begin ? 0 : 1);
        cur += ki1 - ki0;
        return true;
    }
};

// MT = M-tiles of 128 rows that share one dequantised B stage.  With MT = 2 every weight is dequantised
// once per 256 rows instead of once per 128, which halves the dequant work per MMA flop; the two
// accumulators then take both TMEM buffers, so the epilogue only partly overlaps the next tile.
// DG = dequant groups: the DW dequant warps are split into DG teams that fill alternate stages, so the
// dequant of stage s+1 runs beside that of stage s instead of after it.
// KP = MMA issuers per M-tile: with KP = 2 (128-column tiles of one M-tile, which are bound by the ~105 cycles one thread
// needs per tcgen05.mma) a second warp issues the upper two of a K-step's four MMAs into an accumulator of its own, and
// the epilogue adds the two accumulators.
// KS = 64-deep K atoms per pipeline stage: with KS = 2 a stage holds 128 K-elements (one scale group), which halves the
// barrier round trips, waits and commits per K of the small tiles that are bound by them.
// AR = activation rows that a stage holds per 64-deep atom: 128 (a whole M-tile), or 64 when the problem has at most 64
// rows.  The MMA still reads 128 rows; rows 64..127 then alias whatever follows the atom in the stage (the next atom or
// the weight tile: finite or not, they only reach accumulator rows that are never stored).  The 8 KB saved per atom buy
// a deeper pipeline (4 stages of 48 KB instead of 3 of 64 KB), and these problems are bound by the round trip
// stage free -> TMA load / dequant -> MMA -> commit, not by any throughput.
template <int BN, int MT = 1, int DW = 8, int DG = 2, int KP = 1, int KS = 1, int AR = BM>
struct Cfg {
    static_assert(KP == 1 || (KP == 2 && MT == 1 && BN == 128), "K-parity issuers: one M-tile of 128 columns only");
    static_assert(KS == 1 || KS == 2, "one or two 64-deep atoms per stage");
    static_assert(AR == BM || (AR == 64 && MT == 1), "half-height activation atoms: one M-tile only");
    static constexpr int kAAtomBytes = MT * AR * BK * 2;  // one 64-deep atom of the activation tile(s)
    static constexpr int kBAtomBytes = BN * BK * 2;
    static constexpr int kIssuers = MT == 2 ? 2 : KP;
    static constexpr int kGroupWarps = DW / DG;
    // producer, MMA, 4 epilogue and DW dequant warps (16 dequant warps were measured no faster than 8)
    // MT == 2 adds a second MMA-issuing warp (the last one): each issuer owns one M-tile of the pair
    static constexpr int kMmaWarp2 = 6 + DW;
    static constexpr int kThreads = (6 + DW + (kIssuers == 2 ? 1 : 0)) * 32;
    static constexpr int kABytes = kAAtomBytes * KS;  // 16 KB per M-tile and atom
    static constexpr int kBBytes = kBAtomBytes * KS;  // 32 / 16 KB per atom
    static constexpr int kStages = (192 * 1024) / (kABytes + kBBytes);
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN * KP;
    static constexpr int kBlocksPerStage = (BN / 64) * 4 * KS;  // 512-byte packed blocks per stage
    static constexpr int kBlocksPerWarp = kBlocksPerStage / kGroupWarps;
    static_assert(kBlocksPerStage % kGroupWarps == 0 && kGroupWarps % (BN / 64) == 0,
                  "a dequant team must divide the packed blocks of a stage and keep one chunk per warp");
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 4 * 2 * kEpiWarpBytes + 1024;  // + alignment slack
    // instruction descriptor: D fp32, A/B bf16, both K-major, N = BN, M = 128
    static constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                                       (static_cast<uint32_t>(BM >> 4) << 24);
};

template <int NBLK>
struct DequantRegs {
    uint4 w[NBLK];
};

template <int BN, int MT, int DW, int DG, int KP, int KS, int AR>
__global__ void __launch_bounds__((6 + DW + ((MT == 2 || KP == 2) ? 1 : 0)) * 32, 1)
w4a16_prefill_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_c,
                     const __grid_constant__ CUtensorMap tmap_t, const __grid_constant__ CUtensorMap tmap_lb, const PrefillParams p) {
    using C = Cfg<BN, MT, DW, DG, KP, KS, AR>;
    using Regs = DequantRegs<C::kBlocksPerWarp>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + C::kStages * C::kStageBytes;
    auto full_a = [&](int s) { return bar_base + 8u * s; };
    auto full_b = [&](int s) { return bar_base + 8u * s; };  // same barrier as full_a: one wait per K-step for the issuer
    auto empty = [&](int s) { return bar_base + 8u * (2 * C::kStages + s); };
    auto tmem_full = [&](int a) { return bar_base + 8u * (3 * C::kStages + a); };
    auto tmem_empty = [&](int a) { return bar_base + 8u * (3 * C::kStages + 2 + a); };
    const uint32_t epi_base = bar_base + C::kBarrierBytes;
    uint8_t *bar_gen = smem_gen + C::kStages * C::kStageBytes;
    volatile uint32_t *tmem_ptr_slot = reinterpret_cast<volatile uint32_t *>(bar_gen + 8 * (3 * C::kStages + 4));
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(bar_gen + 8 * (3 * C::kStages + 4) + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            // one "stage full" barrier: the TMA producer (1 arrival + the tile's bytes) and the threads of the dequant team
            mbar_init(full_a(s), 1 + C::kGroupWarps * 32);
            mbar_init(empty(s), C::kIssuers);  // one tcgen05.commit per MMA issuer
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full(a), KP);  // one tcgen05.commit per issuer that writes into this buffer
            mbar_init(tmem_empty(a), kNumEpilogueThreads);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t *>(tmem_ptr_slot))),
                     "r"(static_cast<uint32_t>(C::kTmemCols))
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr_slot;
    // Programmatic dependent launch: the next kernel in the stream may start on SMs this grid has left (or never used) and
    // run its prologue and its weight stream there.  In this kernel only the activation loads and every global write
    // order themselves after the previous kernel (griddepcontrol.wait); the packed weights and scales never depend on it.
    pdl_launch_dependents();

    const int chunks_n = p.n >> 6;
    int mt, nt, sp, ki0, ki1, slab;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            pdl_wait();  // the activations may be the previous kernel's output
            uint32_t it = 0;
            bool ok = true;
            WorkIter wi(p);
            while (ok && wi.next(mt, nt, sp, ki0, ki1, slab)) {
                const int ki1e = ki1 + ((KS == 1 && ki0 == 0) ? p.lora_steps : 0);  // + the LoRA steps of the tile
                for (int ki = ki0; ki < ki1e; ++ki, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!(ok = mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, 0x100u | s, p.wait_limit_ns))) break;
                    if (ki >= ki1) {  // LoRA step: both operand tiles come by TMA (rows past m, columns past r read zero)
                        mbar_arrive_expect_tx(full_a(s), C::kAAtomBytes + C::kBAtomBytes);
                        tma_load_2d(smem_base + s * C::kStageBytes, &tmap_t, (ki - ki1) * BK, mt * (BM * MT), full_a(s));
                        tma_load_2d(smem_base + s * C::kStageBytes + C::kABytes, &tmap_lb, (ki - ki1) * BK, nt * BN, full_a(s));
                        continue;
                    }
                    mbar_arrive_expect_tx(full_a(s), C::kABytes);
                    if (static_cast<int>(it) != p.test_drop_a_load)
#pragma unroll
                        for (int at = 0; at < KS; ++at)
                            tma_load_2d(smem_base + s * C::kStageBytes + at * C::kAAtomBytes, &tmap_a, (ki * KS + at) * BK, mt * (BM * MT),
                                        full_a(s));
                }
            }
            if (!ok) {
                // drain: wait (bounded, ignoring the abort flag) for copies already issued
                const uint32_t first = it >= static_cast<uint32_t>(C::kStages) ? it - C::kStages : 0;
                for (uint32_t j = first; j < it; ++j) {
                    const int s = j % C::kStages;
                    const uint32_t ph = (j / C::kStages) & 1;
                    mbar_wait_quiet(full_a(s), ph);
                }
            }
        }
    } else if (warp == 1 || (C::kIssuers == 2 && warp == C::kMmaWarp2)) {
        // ---------------- MMA issuer(s) ----------------
        // One thread issues about one tcgen05.mma per ~105 cycles and spends ~400 more per K-step on the
        // barrier waits and the commit, which is more than the 1024 cycles the eight 128 x 256 x 16 MMAs of a
        // pair execute in.  With MT == 2 the two M-tiles therefore have one issuer each (warp 1: tile 0, the
        // last warp: tile 1); their MMAs go to different accumulators and need no order between them.  With
        // KP == 2 (one M-tile of 128 columns, whose four MMAs per K-step execute in 256 cycles) the two issuers
        // share the K-step instead: warp 1 issues MMAs 0 and 1, the last warp MMAs 2 and 3, each into an
        // accumulator of its own, and the epilogue adds the two (gate+up M=64: 20.6 -> 18.7 us).
        if (lane == 0) {
            const int h0 = (MT == 2 && warp != 1) ? 1 : 0, h1 = MT == 2 ? h0 + 1 : 1;
            const int q = (KP == 2 && warp != 1) ? 1 : 0;  // K-parity issuer: MMAs 2q, 2q+1 of every K-step, accumulator q
            uint32_t it = 0, tile = 0;
            bool ok = true;
            WorkIter wi(p);
            for (; ok && wi.next(mt, nt, sp, ki0, ki1, slab); ++tile) {
                // MT == 1: the two TMEM buffers alternate between tiles.  MT == 2: buffer h holds M-tile h of the pair.
                const uint32_t acc0 = MT == 1 ? (tile & 1) : 0u, acc_ph = MT == 1 ? ((tile >> 1) & 1) : (tile & 1);
                const int ki1e = ki1 + ((KS == 1 && ki0 == 0) ? p.lora_steps : 0);  // + the LoRA steps of the tile
                for (int ki = ki0; ki < ki1e; ++ki, ++it) {
                    const int s = it % C::kStages;
                    const uint32_t ph = (it / C::kStages) & 1;
                    if (!(ok = mbar_wait(full_a(s), ph, abort_flag, p.status, 0x300u | s, p.wait_limit_ns))) break;
                    tc_fence_after();
                    for (int h = h0; h < h1; ++h) {
                        const uint32_t acc = acc0 + h;
                        if (ki == ki0) {  // first write into this accumulator: the epilogue must have drained it
                            if (!(ok = mbar_wait(tmem_empty(acc), acc_ph ^ 1, abort_flag, p.status, 0x200u | acc, p.wait_limit_ns))) break;
                            tc_fence_after();
                        }
                        constexpr int kPer = (BK / 16) * KS / KP;  // MMAs of this issuer per stage and M-tile
#pragma unroll
                        for (int j = 0; j < kPer; ++j) {
                            const int kg = q * kPer + j, at = kg >> 2, kw = kg & 3;  // 64-deep atom, 16-deep slice in it
                            const uint64_t a_desc = make_smem_desc(smem_base + s * C::kStageBytes + at * C::kAAtomBytes + h * (BM * BK * 2));
                            const uint64_t b_desc = make_smem_desc(smem_base + s * C::kStageBytes + C::kABytes + at * C::kBAtomBytes);
                            umma_bf16(tmem_base + (acc * KP + q) * BN, a_desc + 2 * kw, b_desc + 2 * kw, C::kIdesc,
                                      (ki > ki0 || j > 0) ? 1u : 0u);
                        }
                        if (ki == ki1e - 1) umma_commit(tmem_full(acc));  // accumulator h is complete
                    }
                    if (!ok) break;
                    umma_commit(empty(s));  // this issuer's MMAs have read the stage; the slot is free after all issuers'
                }
            }
        }
    } else if (warp < kDequantWarp0) {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
        pdl_wait();  // C (or the workspace) may still be read or written by the previous kernel
        uint32_t tile = 0;
        bool ok = true;
        WorkIter wi(p);
        for (; ok && wi.next(mt, nt, sp, ki0, ki1, slab); ++tile) {
            const uint32_t acc0 = MT == 1 ? (tile & 1) : 0u, acc_ph = MT == 1 ? ((tile >> 1) & 1) : (tile & 1);
#pragma unroll 1
            for (int h = 0; h < MT && ok; ++h) {
            const uint32_t acc = acc0 + h;
            if (!(ok = mbar_wait(tmem_full(acc), acc_ph, abort_flag, p.status, 0x500u | acc, p.wait_limit_ns))) break;
            tc_fence_after();
            const int row = (mt * MT + h) * BM + quarter * 32 + lane;
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * KP * BN;
            if (slab < 0 && p.splits == 1) {
                // bf16 result, 64 columns per round.  A thread owns one row of the accumulator; the 128-byte pieces go
                // through a per-warp shared-memory tile so that the global (or peer, over NVLink) stores are 128
                // contiguous bytes per row and four rows per instruction instead of 16 scattered bytes.  The TMEM loads
                // of round i+1 are issued as soon as the registers of round i are in shared memory, so their latency
                // hides behind the stores, and the accumulator is handed back to the MMA issuer right after the
                // last load has landed, not after the last store.
                // This GPU's own copy of the result (the only copy when the all-gather is not fused) leaves through one
                // asynchronous TMA store of the 32 x 64 tile per round; copies for other GPUs (fused all-gather) are read
                // back from the same tile and stored over NVLink, 128 contiguous bytes of four rows per instruction, or
                // once through the NVSwitch multicast address.
                const bool tma_out = (p.n_peers == 0 && !p.mc_c) || p.self_peer >= 0;
                const bool remote_out = p.mc_c || p.n_peers > (p.self_peer >= 0 ? 1 : 0);
                // two staging tiles per warp, used in turn: the TMA store of one round reads its tile while the next round fills the other
                const uint32_t epi_tma0 = epi_base + static_cast<uint32_t>(warp - 2) * (2 * kEpiWarpBytes);  // 1024-byte aligned swizzle atoms
                const int x0_out = (p.n_peers > 0 ? p.col0 : 0) + nt * BN;  // first column of the tile in the output buffer
                uint32_t ra[32], rb[32];
                if (KP == 1 && p.swiglu) {
                    // SwiGLU (kiln-model/src/forward.rs:2769-2839 as one GEMM): a 64-column run of the tile is 32 gate columns and
                    // their 32 up columns, i.e. the two register buffers of a round; silu(gate) * up is computed in fp32 and
                    // stored straight from registers (64 contiguous bytes per thread and round) while the next round's TMEM
                    // loads are in flight
                    __nv_bfloat16 *crow = p.C + static_cast<size_t>(row) * (p.n >> 1) + ((nt * BN) >> 1);
                    tmem_ld_32x32b_x32(t_row, ra);
                    tmem_ld_32x32b_x32(t_row + 32, rb);
#pragma unroll 1
                    for (int pp = 0; pp < BN / 64; ++pp) {
                        tmem_ld_wait();
                        uint4 *dst = reinterpret_cast<uint4 *>(crow + pp * 32);
#pragma unroll
                        for (int v = 0; v < 4; ++v) {  // eight output columns at a time: their registers die with the store
                            uint32_t o[4];
#pragma unroll
                            for (int e2 = 0; e2 < 4; ++e2) {
                                const int e = 4 * v + e2;
                                float ga = __uint_as_float(ra[2 * e]), gb = __uint_as_float(ra[2 * e + 1]);
                                float ua = __uint_as_float(rb[2 * e]), ub = __uint_as_float(rb[2 * e + 1]);
                                if (p.per_column) {
                                    const int pg = scale_single_pos(nt * BN + pp * 64 + 2 * e), pu = scale_single_pos(nt * BN + pp * 64 + 32 + 2 * e);
                                    ga *= __half2float(p.S[pg]);
                                    gb *= __half2float(p.S[pg + 1]);
                                    ua *= __half2float(p.S[pu]);
                                    ub *= __half2float(p.S[pu + 1]);
                                }
                                __nv_bfloat162 b = __floats2bfloat162_rn(__fdividef(ga, 1.f + __expf(-ga)) * ua, __fdividef(gb, 1.f + __expf(-gb)) * ub);
                                o[e2] = *reinterpret_cast<uint32_t *>(&b);
                            }
                            if (row < p.m) dst[v] = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                        if (pp + 1 < BN / 64) {
                            tmem_ld_32x32b_x32(t_row + (pp + 1) * 64, ra);
                            tmem_ld_32x32b_x32(t_row + (pp + 1) * 64 + 32, rb);
                        } else {
                            tc_fence_before();
                            mbar_arrive(tmem_empty(acc));
                        }
                    }
                    continue;
                }
                if constexpr (KP == 2) {
                    // two accumulators (one per K-parity issuer) to add: 32 columns of each per half-round; the loads of the
                    // next half-round are in flight while a finished 64-column tile is stored
                    tmem_ld_32x32b_x32(t_row, ra);
                    tmem_ld_32x32b_x32(t_row + BN, rb);
#pragma unroll 1
                    for (int hh = 0; hh < BN / 32; ++hh) {
                        const int pp = hh >> 1, half = hh & 1;
                        const uint32_t epi_tma = epi_tma0 + static_cast<uint32_t>(pp & 1) * kEpiWarpBytes;
                        const int col = nt * BN + hh * 32;
                        tmem_ld_wait();
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint32_t o[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float x0 = __uint_as_float(ra[8 * v + 2 * e]) + __uint_as_float(rb[8 * v + 2 * e]);
                                float x1 = __uint_as_float(ra[8 * v + 2 * e + 1]) + __uint_as_float(rb[8 * v + 2 * e + 1]);
                                if (p.per_column) {
                                    const int pos = scale_single_pos(col + 8 * v + 2 * e);
                                    x0 *= __half2float(p.S[pos]);
                                    x1 *= __half2float(p.S[pos + 1]);
                                }
                                __nv_bfloat162 b = __floats2bfloat162_rn(x0, x1);
                                o[e] = *reinterpret_cast<uint32_t *>(&b);
                            }
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                                             epi_tma + lane * 128 + (((half * 4 + v) ^ (lane & 7)) << 4)),
                                         "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                         : "memory");
                        }
                        if (hh + 1 < BN / 32) {
                            tmem_ld_32x32b_x32(t_row + (hh + 1) * 32, ra);
                            tmem_ld_32x32b_x32(t_row + BN + (hh + 1) * 32, rb);
                        } else {
                            tc_fence_before();
                            mbar_arrive(tmem_empty(acc));  // every column of both accumulators is in registers or shared memory
                        }
                        if (half == 0) continue;
                        if (tma_out) fence_proxy_async_smem();
                        __syncwarp();
                        if (tma_out && lane == 0) {
                            tma_store_2d(&tmap_c, epi_tma, x0_out + pp * 64, (mt * MT + h) * BM + quarter * 32);
                            bulk_commit_group();
                        }
                        if (remote_out) {
                            const int piece = lane & 7;
                            const int col_out = p.col0 + nt * BN + pp * 64 + piece * 8;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const int rl = i * 4 + (lane >> 3);
                                const int grow = (mt * MT + h) * BM + quarter * 32 + rl;
                                uint4 val;
                                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                             : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                             : "r"(epi_tma + rl * 128 + ((piece ^ (rl & 7)) << 4)));
                                if (grow < p.m) {
                                    if (p.mc_c) {
                                        asm volatile("multimem.st.weak.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(
                                                         p.mc_c + static_cast<size_t>(grow) * p.ldc + col_out),
                                                     "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w)
                                                     : "memory");
                                    } else {
                                        for (int pe = 0; pe < p.n_peers; ++pe)
                                            if (pe != p.self_peer)
                                                *reinterpret_cast<uint4 *>(p.peer_c[pe] + static_cast<size_t>(grow) * p.ldc + col_out) = val;
                                    }
                                }
                            }
                        }
                        if (tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        __syncwarp();
                    }
                    continue;  // the accumulators were released above
                }
                tmem_ld_32x32b_x32(t_row, ra);
                tmem_ld_32x32b_x32(t_row + 32, rb);
#pragma unroll 1
                for (int pp = 0; pp < BN / 64; ++pp) {
                    const uint32_t epi_tma = epi_tma0 + static_cast<uint32_t>(pp & 1) * kEpiWarpBytes;
                    tmem_ld_wait();
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int col = nt * BN + pp * 64 + half * 32;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            uint32_t o[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float x0 = __uint_as_float(half ? rb[8 * v + 2 * e] : ra[8 * v + 2 * e]);
                                float x1 = __uint_as_float(half ? rb[8 * v + 2 * e + 1] : ra[8 * v + 2 * e + 1]);
                                if (p.per_column) {
                                    const int pos = scale_single_pos(col + 8 * v + 2 * e);
                                    x0 *= __half2float(p.S[pos]);
                                    x1 *= __half2float(p.S[pos + 1]);
                                }
                                __nv_bfloat162 b = __floats2bfloat162_rn(x0, x1);
                                o[e] = *reinterpret_cast<uint32_t *>(&b);
                            }
                            // 128-byte rows, 16-byte chunk index XOR (row % 8): the layout of the 128B-swizzled tensor map
                            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(
                                             epi_tma + lane * 128 + (((half * 4 + v) ^ (lane & 7)) << 4)),
                                         "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3])
                                         : "memory");
                        }
                    }
                    if (pp + 1 < BN / 64) {
                        tmem_ld_32x32b_x32(t_row + (pp + 1) * 64, ra);
                        tmem_ld_32x32b_x32(t_row + (pp + 1) * 64 + 32, rb);
                    } else {
                        tc_fence_before();
                        mbar_arrive(tmem_empty(acc));  // every column of this accumulator is in registers or shared memory
                    }
                    if (tma_out) fence_proxy_async_smem();
                    __syncwarp();
                    if (tma_out && lane == 0) {
                        // (full 128-byte lines, no load back from shared memory; rows past m are clipped by the tensor map)
                        tma_store_2d(&tmap_c, epi_tma, x0_out + pp * 64, (mt * MT + h) * BM + quarter * 32);
                        bulk_commit_group();
                    }
                    if (remote_out) {
                        const int piece = lane & 7;
                        const int col_out = p.col0 + nt * BN + pp * 64 + piece * 8;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rl = i * 4 + (lane >> 3);
                            const int grow = (mt * MT + h) * BM + quarter * 32 + rl;
                            uint4 val;
                            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                         : "r"(epi_tma + rl * 128 + ((piece ^ (rl & 7)) << 4)));
                            if (grow < p.m) {
                                if (p.mc_c) {
                                    asm volatile("multimem.st.weak.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(
                                                     p.mc_c + static_cast<size_t>(grow) * p.ldc + col_out),
                                                 "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w)
                                                 : "memory");
                                } else {
                                    // column-parallel all-gather fused into the epilogue: plain stores into the other GPUs' buffers
                                    for (int pe = 0; pe < p.n_peers; ++pe)
                                        if (pe != p.self_peer)
                                            *reinterpret_cast<uint4 *>(p.peer_c[pe] + static_cast<size_t>(grow) * p.ldc + col_out) = val;
                                }
                            }
                        }
                    }
                    // this tile is rewritten two rounds from now: the TMA store of the round before this one has read the
                    // other tile (the next round's TMEM loads are already in flight), and every lane is done with this one
                    if (tma_out && lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    __syncwarp();
                }
                continue;  // the accumulator was released above
            }
#pragma unroll 1
            for (int cc = 0; cc < BN / 32; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(t_row + cc * 32, r);
                if constexpr (KP == 2) {  // add the second K-parity accumulator
                    uint32_t r2[32];
                    tmem_ld_32x32b_x32(t_row + BN + cc * 32, r2);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(r2[i]));
                }
                tmem_ld_wait();
                if (slab >= 0) {
                    // stream-K piece: tile-shaped fp32 slab, all rows (rows past m hold zeros)
                    float4 *dst = reinterpret_cast<float4 *>(p.partial + static_cast<size_t>(slab) * p.tile_elems +
                                                             static_cast<size_t>(h * BM + quarter * 32 + lane) * BN + cc * 32);
#pragma unroll
                    for (int v = 0; v < 8; ++v)
                        dst[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                             __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                } else if (row < p.m) {
                    const int col = nt * BN + cc * 32;
                    {
                        float4 *dst = reinterpret_cast<float4 *>(
                            p.partial + (static_cast<size_t>(sp) * p.m + row) * p.n + col);
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            dst[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                                 __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(tmem_empty(acc));
            }
        }
        if (lane == 0) bulk_wait_group0();  // this warp's TMA stores are complete before the CTA may exit
    } else {
        // ---------------- dequant: packed int4 -> bf16 B tile ----------------
        const int dw = (warp - kDequantWarp0) / DG, team = (warp - kDequantWarp0) % DG;  // warp `dw` of team `team`
        const int qd = lane & 3, c = lane >> 2;
        constexpr int kChunksPerTile = BN / 64;
        uint32_t it_base = 0;  // stages issued before this piece of work (all teams count alike)
        bool ok = true;
        int cur_group = -1;
        uint32_t s2[8];  // bf16x2 {s, s} for columns 8t + c of this warp's chunk
        WorkIter wi(p);
        while (ok && wi.next(mt, nt, sp, ki0, ki1, slab)) {
            cur_group = -1;
            auto load_regs = [&](Regs &d, int ki) {
#pragma unroll
                for (int b = 0; b < C::kBlocksPerWarp; ++b) {
                    const int blk = dw + C::kGroupWarps * b;
                    const int ch = blk % kChunksPerTile, kt = blk / kChunksPerTile;
                    const size_t idx =
                        (static_cast<size_t>(ki * (4 * KS) + kt) * chunks_n + nt * kChunksPerTile + ch) * 32 + lane;
                    d.w[b] = ld_stream_v4(p.B + idx);
                }
            };
            auto group_of = [](int ki) { return KS == 2 ? ki : (ki >> 1); };  // scale group of a stage (KS == 2: a stage is a group)
            auto load_scales = [&](int g) {
                return ld_stream_v4(reinterpret_cast<const uint4 *>(
                    p.S + static_cast<size_t>(g) * p.n + (nt * kChunksPerTile + dw % kChunksPerTile) * 64 + 8 * c));
            };
            // this team's K-steps of the piece: those whose stage number is congruent to `team`
            const int kf = ki0 + static_cast<int>((static_cast<uint32_t>(team) + DG - it_base % DG) % DG);
            // Packed words and scales of this team's next three K-steps are always in flight, each step's in registers of
            // its own: the loop below is unrolled three times so that no register with a pending load is ever copied (a
            // copy would wait for the load and shrink the three round trips in flight to one).
            Regs rw[3];
            uint4 rs[3];
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                rs[u] = make_uint4(0, 0, 0, 0);
                if (kf + u * DG < ki1) {
                    load_regs(rw[u], kf + u * DG);
                    if (!p.per_column) rs[u] = load_scales(group_of(kf + u * DG));
                }
            }
            for (int kb = kf; kb < ki1 && ok; kb += 3 * DG) {
#pragma unroll
            for (int u = 0; u < 3; ++u) {
                const int ki = kb + u * DG;
                if (ki >= ki1) break;
                Regs &r0 = rw[u];
                const uint32_t it = it_base + static_cast<uint32_t>(ki - ki0);
                const int s = it % C::kStages;
                const uint32_t ph = (it / C::kStages) & 1;
                // scales of this K-step's group (all blocks of a warp share one chunk: blk % kChunksPerTile == dw % ..)
                const int g = p.per_column ? 0 : group_of(ki);
                if (g != cur_group) {
                    cur_group = g;
                    if (p.per_column) {
#pragma unroll
                        for (int t = 0; t < 8; ++t) s2[t] = 0x3F803F80u;  // bf16x2 {1, 1}; scale applied in the epilogue
                    } else {
                        const uint32_t sw[4] = {rs[u].x, rs[u].y, rs[u].z, rs[u].w};
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const float f = __half2float(__ushort_as_half(
                                static_cast<unsigned short>((t & 1) ? (sw[t >> 1] >> 16) : (sw[t >> 1] & 0xFFFFu))));
                            __nv_bfloat162 b = __floats2bfloat162_rn(f, f);
                            s2[t] = *reinterpret_cast<uint32_t *>(&b);
                        }
                    }
                }
                if (!(ok = mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, 0x600u | s, p.wait_limit_ns))) break;
                const uint32_t b_tile = smem_base + s * C::kStageBytes + C::kABytes;
#pragma unroll
                for (int b = 0; b < C::kBlocksPerWarp; ++b) {
                    const int blk = dw + C::kGroupWarps * b;
                    const int ch = blk % kChunksPerTile, ktb = blk / kChunksPerTile;  // 16-row K tile of the stage: 0 .. 4*KS-1
                    const int at = ktb >> 2, kt = ktb & 3;                            // 64-deep atom, K tile inside it
                    const uint32_t xs[4] = {r0.w[b].x, r0.w[b].y, r0.w[b].z, r0.w[b].w};
                    // row (= column of B) n_local = ch*64 + 8t + c, 128 B per row; 16-byte chunk (2kt + half) ^ c
                    const uint32_t row_base = b_tile + static_cast<uint32_t>(at * C::kBAtomBytes) + static_cast<uint32_t>(ch * 64 + c) * 128u + 4u * qd;
                    const uint32_t sw_lo = static_cast<uint32_t>((2 * kt) ^ c) << 4;
                    const uint32_t sw_hi = static_cast<uint32_t>((2 * kt + 1) ^ c) << 4;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t x = xs[j];
                        uint32_t v[4];
                        v[0] = lop3_and_or(x, kNibMask, kMagic128);        // K 2qd, 2qd+1     col 16j + c
                        v[1] = lop3_and_or(x >> 4, kNibMask, kMagic128);   // K 2qd+8, 2qd+9   col 16j + c
                        v[2] = lop3_and_or(x >> 8, kNibMask, kMagic128);   // K 2qd, 2qd+1     col 16j + 8 + c
                        v[3] = lop3_and_or(x >> 12, kNibMask, kMagic128);  // K 2qd+8, 2qd+9   col 16j + 8 + c
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            __nv_bfloat162 w = *reinterpret_cast<__nv_bfloat162 *>(&v[e]);
                            const uint32_t k136 = kPos136x2;
                            w = __hsub2(w, *reinterpret_cast<const __nv_bfloat162 *>(&k136));
                            w = __hmul2(w, *reinterpret_cast<const __nv_bfloat162 *>(&s2[2 * j + (e >> 1)]));
                            v[e] = *reinterpret_cast<uint32_t *>(&w);
                        }
                        const uint32_t r_lo = row_base + static_cast<uint32_t>(16 * j) * 128u;
                        const uint32_t r_hi = r_lo + 8u * 128u;
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(r_lo + sw_lo), "r"(v[0]) : "memory");
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(r_lo + sw_hi), "r"(v[1]) : "memory");
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(r_hi + sw_lo), "r"(v[2]) : "memory");
                        asm volatile("st.shared.b32 [%0], %1;" ::"r"(r_hi + sw_hi), "r"(v[3]) : "memory");
                    }
                }
                // every thread publishes its own stores to the async proxy and arrives itself (one arrival per
                // warp behind a __syncwarp was measured slower: 1154 vs 1217 TFLOP/s on gate+up M=8192)
                fence_proxy_async_smem();
                mbar_arrive(full_b(s));
                if (ki + 3 * DG < ki1) {
                    load_regs(rw[u], ki + 3 * DG);
                    if (!p.per_column) rs[u] = load_scales(group_of(ki + 3 * DG));
                }
            }
            }
            it_base += static_cast<uint32_t>(ki1 - ki0);
            // LoRA steps of the tile: the weight-side tile comes by TMA; the team that owns a stage only owes its barrier the arrivals
            if (KS == 1 && ki0 == 0 && p.lora_steps > 0) {
                for (int e = 0; e < p.lora_steps && ok; ++e, ++it_base) {
                    if (it_base % DG != static_cast<uint32_t>(team)) continue;
                    const int s = it_base % C::kStages;
                    const uint32_t ph = (it_base / C::kStages) & 1;
                    if (!(ok = mbar_wait(empty(s), ph ^ 1, abort_flag, p.status, 0x700u | s, p.wait_limit_ns))) break;
                    mbar_arrive(full_b(s));
                }
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(static_cast<uint32_t>(C::kTmemCols))
                     : "memory");
    }
}

// out[m][n] = bf16(sum_s partial[s][m][n]) (* per-column scale)
__global__ void splitk_reduce_kernel(const float *partial, __nv_bfloat16 *C, const __half *S, int m, int n,
                                     int splits, int per_column) {
    pdl_launch_dependents();
    pdl_wait();  // the partial sums come from the kernel launched just before
    const size_t total4 = static_cast<size_t>(m) * n / 4;
    const size_t slab4 = total4;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total4;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 acc = reinterpret_cast<const float4 *>(partial)[i];
        for (int s = 1; s < splits; ++s) {
            const float4 v = reinterpret_cast<const float4 *>(partial)[i + s * slab4];
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        if (per_column) {
            const int col = static_cast<int>((i * 4) % n);
            const int p0 = scale_single_pos(col), p1 = scale_single_pos(col + 2);
            acc.x *= __half2float(S[p0]);
            acc.y *= __half2float(S[p0 + 1]);
            acc.z *= __half2float(S[p1]);
            acc.w *= __half2float(S[p1 + 1]);
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        reinterpret_cast<uint2 *>(C)[i] = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
    }
}

// Stream-K fix-up: gridDim.y blocks per output tile of the remainder.  Recomputes which CTAs covered only a part of
// the tile's K-steps (the same arithmetic as WorkIter), sums their slabs in CTA order and writes bf16.  A tile that
// one CTA covered completely was already written by that CTA.
__global__ void streamk_fixup_kernel(const float *partial, __nv_bfloat16 *C, const __half *S, int m, int n, int m_tiles,
                                     int k_iters, int tile_rows, int bn, int ctas, long long total, int first_tile,
                                     int per_column) {
    pdl_launch_dependents();
    pdl_wait();  // the slabs come from the kernel launched just before
    const int tr = blockIdx.x;
    const long long t0 = static_cast<long long>(tr) * k_iters, t1 = t0 + k_iters;
    int r_lo = static_cast<int>(t0 * ctas / total) - 1, r_hi = static_cast<int>(t1 * ctas / total) + 1;
    if (r_lo < 0) r_lo = 0;
    if (r_hi > ctas - 1) r_hi = ctas - 1;
    int slabs[40];
    int ns = 0;
    for (int r = r_lo; r <= r_hi; ++r) {
        const long long g0 = total * r / ctas, g1 = total * (r + 1) / ctas;
        const long long a = g0 > t0 ? g0 : t0, b = g1 < t1 ? g1 : t1;
        if (a >= b) continue;
        if (a == t0 && b == t1) return;  // whole tile by one CTA: nothing to fix up
        if (ns < 40) slabs[ns++] = 2 * r + (a == g0 ? 0 : 1);
    }
    const int t = first_tile + tr;
    const int mt = t % m_tiles, nt = t / m_tiles;
    const size_t tile_elems = static_cast<size_t>(tile_rows) * bn;
    const int vec_per_row = bn / 4;
    // gridDim.y blocks share a tile by rows
    const int rows_per_block = (tile_rows + gridDim.y - 1) / gridDim.y;
    const int r_begin = blockIdx.y * rows_per_block;
    for (int i = threadIdx.x; i < rows_per_block * vec_per_row; i += blockDim.x) {
        const int rl = r_begin + i / vec_per_row, cv = i % vec_per_row;
        if (rl >= tile_rows) break;
        const int row = mt * tile_rows + rl;
        if (row >= m) continue;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < ns; ++j) {
            const float4 v = *reinterpret_cast<const float4 *>(partial + slabs[j] * tile_elems +
                                                               static_cast<size_t>(rl) * bn + 4 * cv);
            acc.x += v.x;
            acc.y += v.y;
            acc.z += v.z;
            acc.w += v.w;
        }
        const int col = nt * bn + 4 * cv;
        if (per_column) {
            const int p0 = scale_single_pos(col), p1 = scale_single_pos(col + 2);
            acc.x *= __half2float(S[p0]);
            acc.y *= __half2float(S[p0 + 1]);
            acc.z *= __half2float(S[p1]);
            acc.w *= __half2float(S[p1 + 1]);
        }
        __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
        *reinterpret_cast<uint2 *>(C + static_cast<size_t>(row) * n + col) =
            make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
    }
}

// ---- host -----------------------------------------------------------------------------------

struct PrefillConfig {
    int bn, splits, mt, stream_k;
};

// Cost model of one launch, least-squares fitted (mean error 6 %) to 1100 timed launches on B200: 5 projection shapes x
// M = 64..8192 x every tiling the rule considers, each timed alone after an L2 flush.  Microseconds:
//   launch + waves * (K-steps per unit * step + tile) [+ split-K: fixed + per MB of fp32 slab traffic]
//   stream-K: launch + whole waves as above + share * step + 2 * tile + per MB of remainder tiles + per slab piece
// `step` is the time of one 64-K step of a CTA, `tile` what a tile adds on top (epilogue that does not overlap, pipeline
// restart); both depend on the columns per tile and the M-tiles per stage.  On the fitted set the model's choice is
// within 0.3 % of the best measured tiling in total.
struct TileCost {
    double step, tile;
};
TileCost tile_cost(int bn, int mt) {
    if (mt == 2) return bn == 256 ? TileCost{0.584, 11.26} : TileCost{0.463, 3.83};
    return bn == 256 ? TileCost{0.489, 4.85} : TileCost{0.301, 2.10};
}
constexpr double kCostLaunch = 7.02, kCostSplitFixed = 4.21, kCostSplitPerMB = 0.332, kCostSkPerMB = 0.177, kCostSkPerPiece = 0.147;

// Stream-K split of `tiles` tiles over `grid` CTAs: the tiles of the whole waves are dealt round-robin, the K-steps of
// the rest go in equal shares to `ctas` CTAs.  A share is at least 8 K-steps and at least 1/36 of a tile, so that no tile
// is spread over more slabs than the fix-up kernel sums (40).
struct StreamKPlan {
    int first_tile, ctas;
};
StreamKPlan streamk_plan(int tiles, int k_iters, int grid) {
    StreamKPlan pl;
    pl.first_tile = tiles / grid * grid;
    const long long total = static_cast<long long>(tiles - pl.first_tile) * k_iters;
    const int min_share = k_iters / 36 + 1 > 8 ? k_iters / 36 + 1 : 8;
    long long c = total / min_share;
    pl.ctas = static_cast<int>(c > grid ? grid : (c < 1 ? 1 : c));
    return pl;
}

PrefillConfig g_prefill_override{0, 0, 0, 0};
unsigned long long g_wait_limit_ns = kWaitLimitNs;
int g_test_drop_a_load = -1;
int g_smallm_enabled = 1;

PrefillConfig choose_prefill(int m, int n, int k, bool allow_pairs = true, bool allow_scratch = true,
                             size_t max_split_bytes = ~static_cast<size_t>(0)) {
    const int sms = device_sm_count();
    const int k_iters = k / BK;
    {  // tuning hook (kiln_w4a16_set_prefill_override): taken when it is legal for this problem, else the rule below
        const PrefillConfig &o = g_prefill_override;
        const bool legal = (o.bn == 128 || o.bn == 256) && n % o.bn == 0 && (o.mt == 1 || (o.mt == 2 && allow_pairs && m > BM)) &&
                           o.splits >= 1 && o.splits <= 8 && k_iters / o.splits >= 1 && (o.stream_k == 0 || o.stream_k == 1) &&
                           !(o.stream_k && o.splits != 1) && (allow_scratch || (o.splits == 1 && !o.stream_k));
        // (a forced split larger than max_split_bytes is returned as it is: the no-allocation entry then refuses the call)
        if (legal) return o;
    }
    PrefillConfig best{256, 1, 1, 0};
    double best_t = 1e30;
    const int bns[2] = {256, 128};
    const int ss[6] = {1, 2, 3, 4, 6, 8};
    for (int mt = 1; mt <= (allow_pairs ? 2 : 1); ++mt)
        for (int bi = 0; bi < 2; ++bi)
            for (int si = 0; si < 6; ++si) {
                const int bn = bns[bi], s = ss[si];
                if (k_iters / s < 8) continue;
                if (s > 1 && !allow_scratch) continue;
                if (s > 1 && static_cast<size_t>(s) * m * n * sizeof(float) > max_split_bytes) continue;
                if (mt == 2 && m <= BM) continue;
                const int m_tiles = (m + BM * mt - 1) / (BM * mt);
                const long long units = static_cast<long long>(m_tiles) * (n / bn) * s;
                const double waves = static_cast<double>((units + sms - 1) / sms);
                const TileCost tc = tile_cost(bn, mt);
                double t = kCostLaunch + waves * (static_cast<double>(k_iters) / s * tc.step + tc.tile);
                if (s > 1) t += kCostSplitFixed + kCostSplitPerMB * (static_cast<double>(s) + 0.5) * m * static_cast<double>(n) * 4.0 / 1.0e6;
                if (t < best_t) {
                    best_t = t;
                    best = PrefillConfig{bn, s, mt, 0};
                }
                // hybrid stream-K over the same tiling: whole waves as above, the remaining tiles' K-steps in equal
                // shares, plus the fix-up pass over those tiles
                if (s == 1 && allow_pairs && allow_scratch) {  // (the no-alloc entry, which passes allow_pairs = false, has no fix-up pass)
                    const long long tiles = static_cast<long long>(m_tiles) * (n / bn);
                    const StreamKPlan pl = streamk_plan(static_cast<int>(tiles), k_iters, sms);
                    const long long rem = tiles - pl.first_tile;
                    if (rem > 0 && rem < sms) {
                        const double share = static_cast<double>(rem) * k_iters / pl.ctas;
                        const double tile_mb = BM * mt * bn * 4.0 / 1.0e6;
                        const double tk = kCostLaunch + static_cast<double>(pl.first_tile / sms) * (k_iters * tc.step + tc.tile) +
                                          share * tc.step + 2.0 * tc.tile + kCostSkPerMB * static_cast<double>(rem) * tile_mb +
                                          kCostSkPerPiece * static_cast<double>(rem) * k_iters / share;
                        if (tk < best_t) {
                            best_t = tk;
                            best = PrefillConfig{bn, 1, mt, 1};
                        }
                    }
                }
            }
    return best;
}

// Tensor map of the bf16 result [m, n] for the epilogue's TMA stores: boxes of 32 rows x 64 columns, 128-byte swizzle.
bool encode_c_map(EncodeTiledFn enc, CUtensorMap *map, void *c, int m, int n) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(n) * 2};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int MT = 1, int DW = 8, int DG = 2, int KP = 1, int KS = 1, int AR = BM>
int launch_bn(const CUtensorMap &tmap, const CUtensorMap &tmap_c, PrefillParams p, cudaStream_t stream,
              const CUtensorMap *tmap_t = nullptr, const CUtensorMap *tmap_lb = nullptr) {
    using C = Cfg<BN, MT, DW, DG, KP, KS, AR>;
    p.k_iters /= KS;  // the kernel counts pipeline stages of KS atoms (k is a multiple of 128)
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        if (int rc = record_cuda_error(cudaFuncSetAttribute(w4a16_prefill_kernel<BN, MT, DW, DG, KP, KS, AR>,
                                                            cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes)))
            return rc;
        attr_set[dev] = true;
    }
    const int units = p.m_tiles * p.n_tiles * p.splits;
    const int grid = p.stream_k ? device_sm_count() : (units < device_sm_count() ? units : device_sm_count());
    note_launch();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(C::kThreads);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr = pdl_attribute();
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    static const CUtensorMap kNoMap = {};  // (never dereferenced when p.lora_steps == 0)
    if (!tmap_t || !tmap_lb || KS != 1) p.lora_steps = 0;
    return record_cuda_error(cudaLaunchKernelEx(&cfg, w4a16_prefill_kernel<BN, MT, DW, DG, KP, KS, AR>, tmap, tmap_c,
                                                tmap_t ? *tmap_t : kNoMap, tmap_lb ? *tmap_lb : kNoMap, p));
}

}  // namespace

// SwiGLU can be fused into the tcgen05 kernel's epilogue when its tiling for the problem writes whole tiles as bf16.
// whether the small-batch kernel runs a plain problem that the planner tiled as `c`
static bool smallm_takes(const PrefillConfig &c, int m, int n, int k, int groupsize) {
    return g_smallm_enabled && g_test_drop_a_load < 0 && c.bn == 128 && c.mt == 1 && !c.stream_k && c.splits <= k / 128 &&
           smallm_supported(m, n, k, groupsize);
}

bool prefill_fuses_swiglu(int m, int n, int k) {
    const PrefillConfig c = choose_prefill(m, n, k);
    if (c.splits == 1 && smallm_takes(c, m, n, k, 128)) return true;  // (its epilogue pairs the gate and up warps)
    // (not the 128-column tiles of one M-tile: their two K-parity accumulators would have to be added first, and at those
    // batch sizes a second pass over the small output costs less than a longer epilogue)
    return c.splits == 1 && !c.stream_k && !(c.bn == 128 && c.mt == 1);
}

// The LoRA delta can ride in the tcgen05 kernel as extra K-steps unless the scales are per column (those are applied to
// the whole accumulator in the epilogue and would scale the delta too).
bool prefill_fuses_lora(int groupsize, int lora_r) { return groupsize == 128 && lora_r > 0 && lora_r <= 128 && lora_r % 8 == 0; }

void set_wait_limit_ns(unsigned long long ns) { g_wait_limit_ns = ns ? ns : kWaitLimitNs; }
unsigned long long current_wait_limit_ns() { return g_wait_limit_ns; }
void set_smallm_enabled(int on) { g_smallm_enabled = on; }
void set_test_drop_a_load(int k_step) { g_test_drop_a_load = k_step; }

void set_prefill_override(int bn, int splits, int mt, int stream_k) {
    g_prefill_override = PrefillConfig{bn, splits, mt, stream_k};
}

void prefill_plan(int m, int n, int k, int out[4]) {
    const PrefillConfig c = choose_prefill(m, n, k);
    out[0] = c.bn;
    out[1] = c.splits;
    out[2] = c.mt;
    out[3] = c.stream_k;
}

bool prefill_supported(int m, int n, int k, int groupsize) {
    (void)groupsize;
    return m >= 1 && n % 256 == 0 && k % 128 == 0 && k / BK >= 2;
}

size_t workspace_for(const PrefillConfig &c, int m, int n) {
    if (c.stream_k) return static_cast<size_t>(2) * device_sm_count() * (BM * c.mt) * c.bn * sizeof(float);
    return c.splits > 1 ? static_cast<size_t>(c.splits) * m * n * sizeof(float) : 0;
}

size_t prefill_workspace_bytes(int m, int n, int k) { return workspace_for(choose_prefill(m, n, k), m, n); }

int launch_prefill(const GemmArgs &a) {
    EncodeTiledFn enc = encode_fn();
    if (!enc) return KILN_W4A16_ERR_CUDA;
    uint32_t *status = device_status_word();
    if (!status) return KILN_W4A16_ERR_CUDA;
    const bool fused = a.n_peers > 0 || a.mc_c;  // the peer-store epilogue needs whole tiles: no split-K, no stream-K
    const PrefillConfig c = choose_prefill(a.m, a.n, a.k, true, !fused && !a.no_scratch);
    // At most 128 rows in 128-column tiles: the kernel that keeps the dequantised weights in tensor memory (same tiling,
    // same K splits and workspace, so everything the planner reports holds for it too)
    const bool smallm = smallm_takes(c, a.m, a.n, a.k, a.groupsize) && !fused && (!a.swiglu || c.splits == 1) &&
                        (a.lora_r == 0 || (a.lora_t && a.lora_b && prefill_fuses_lora(a.groupsize, a.lora_r)));
    if (!smallm && a.swiglu && (fused || c.splits != 1 || c.stream_k || (c.bn == 128 && c.mt == 1)))
        return KILN_W4A16_ERR_KERN_SHAPE;  // (callers ask prefill_fuses_swiglu first)
    if (smallm) {
        const size_t need = workspace_for(c, a.m, a.n);
        if (need > 0 && (!a.workspace || a.workspace_bytes < need)) return KILN_W4A16_ERR_WORKSPACE;
        int rc = launch_smallm(a, c.splits, static_cast<float *>(a.workspace));
        if (rc == 0 && c.splits > 1) {
            const size_t total4 = static_cast<size_t>(a.m) * a.n / 4;
            int blocks = static_cast<int>((total4 + 255) / 256);
            const int cap = device_sm_count() * 8;
            if (blocks > cap) blocks = cap;
            note_launch();
            rc = record_cuda_error(launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), a.stream, static_cast<float *>(a.workspace),
                                              static_cast<__nv_bfloat16 *>(a.C), static_cast<const __half *>(a.S), a.m, a.n, c.splits,
                                              a.groupsize == -1 ? 1 : 0));
        }
        return rc;
    }

    CUtensorMap tmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(a.k), static_cast<cuuint64_t>(a.m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(a.k) * 2};
    // at most 64 rows in 128-column tiles of one M-tile: half-height activation atoms (AR = 64)
    const bool half_a = a.m <= 64 && c.mt == 1 && c.bn == 128;
    const cuuint32_t box[2] = {BK, static_cast<cuuint32_t>(half_a ? 64 : BM * c.mt)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.A), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return KILN_W4A16_ERR_CUDA;
    // Which of the fused all-gather's buffers lives on this GPU: that copy leaves through the TMA-store path.
    int self_peer = -1;
    if (a.n_peers > 0) {
        int dev = -1, found = 0;
        cudaGetDevice(&dev);
        for (int i = 0; i < a.n_peers && i < 8; ++i) {
            cudaPointerAttributes at;
            if (cudaPointerGetAttributes(&at, a.peer_c[i]) == cudaSuccess && at.type == cudaMemoryTypeDevice && at.device == dev) {
                self_peer = i;
                ++found;
            }
        }
        cudaGetLastError();  // (an unregistered pointer only means "not ours")
        if (found != 1) self_peer = -1;  // ambiguous: every copy goes through the store path of the remote copies
    }
    CUtensorMap tmap_c;  // this GPU's own C: [m, n], or its [m, ldc] buffer of the fused all-gather
    if (self_peer >= 0) {
        if (!encode_c_map(enc, &tmap_c, a.peer_c[self_peer], a.m, a.ldc)) return KILN_W4A16_ERR_CUDA;
    } else if (!encode_c_map(enc, &tmap_c, a.C, a.m, a.swiglu ? a.n / 2 : a.n)) {
        return KILN_W4A16_ERR_CUDA;
    }

    PrefillParams p{};
    p.B = static_cast<const uint4 *>(a.B);
    p.S = static_cast<const __half *>(a.S);
    p.C = static_cast<__nv_bfloat16 *>(a.C);
    p.partial = static_cast<float *>(a.workspace);
    p.status = status;
    p.m = a.m;
    p.n = a.n;
    p.k = a.k;
    p.m_tiles = (a.m + BM * c.mt - 1) / (BM * c.mt);
    p.n_tiles = a.n / c.bn;
    p.splits = c.splits;
    p.k_iters = a.k / BK;
    p.per_column = a.groupsize == -1;
    p.n_peers = a.n_peers;
    p.ldc = a.ldc;
    p.col0 = a.col0;
    p.self_peer = self_peer;
    p.swiglu = a.swiglu;
    // LoRA delta fused as extra K-steps: t = scale * x * A^T (bf16 [m, r], written by the kernel launched just before) and
    // lora_b (bf16 [n, r]) are operand tiles like any other; columns past r read zero
    CUtensorMap tmap_t, tmap_lb;
    const bool lora = a.lora_r > 0 && a.lora_t && a.lora_b;
    if (lora) {
        if (a.groupsize == -1 || a.lora_r % 8 != 0 || a.lora_r > 128) return KILN_W4A16_ERR_KERN_SHAPE;  // (callers ask prefill_fuses_lora first)
        const cuuint64_t td[2] = {static_cast<cuuint64_t>(a.lora_r), static_cast<cuuint64_t>(a.m)};
        const cuuint64_t ld[2] = {static_cast<cuuint64_t>(a.lora_r), static_cast<cuuint64_t>(a.n)};
        const cuuint64_t st[1] = {static_cast<cuuint64_t>(a.lora_r) * 2};
        const cuuint32_t tb[2] = {BK, static_cast<cuuint32_t>(half_a ? 64 : BM * c.mt)}, lb[2] = {BK, static_cast<cuuint32_t>(c.bn)};
        if (enc(&tmap_t, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.lora_t), td, st, tb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS ||
            enc(&tmap_lb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(a.lora_b), ld, st, lb, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return KILN_W4A16_ERR_CUDA;
        p.lora_steps = (a.lora_r + BK - 1) / BK;
    }
    const CUtensorMap *pt = lora ? &tmap_t : nullptr, *plb = lora ? &tmap_lb : nullptr;
    p.mc_c = static_cast<__nv_bfloat16 *>(a.mc_c);
    for (int i = 0; i < a.n_peers && i < 8; ++i) p.peer_c[i] = static_cast<__nv_bfloat16 *>(a.peer_c[i]);
    p.stream_k = c.stream_k;
    p.wait_limit_ns = g_wait_limit_ns;
    p.test_drop_a_load = g_test_drop_a_load;
    p.tile_elems = BM * c.mt * c.bn;
    const StreamKPlan plan = streamk_plan(p.m_tiles * p.n_tiles, p.k_iters, device_sm_count());
    p.sk_first_tile = plan.first_tile;
    p.sk_ctas = plan.ctas;
    const size_t need = workspace_for(c, a.m, a.n);
    if (need > 0 && (!a.workspace || a.workspace_bytes < need)) return KILN_W4A16_ERR_WORKSPACE;

    int rc;
    if (c.mt == 2)
        rc = c.bn == 256 ? launch_bn<256, 2>(tmap, tmap_c, p, a.stream, pt, plb) : launch_bn<128, 2>(tmap, tmap_c, p, a.stream, pt, plb);
    else
        // (128-column tiles of one M-tile are bound by the MMA issue rate: two issuers, each with an accumulator of its own)
        // ... and 128-deep pipeline stages, which halve their barrier round trips per K (not with stream-K, whose fix-up pass
        // counts 64-deep steps, nor when a split would be left without a whole stage)
        if (c.bn == 256)
            rc = launch_bn<256, 1>(tmap, tmap_c, p, a.stream, pt, plb);
        else if (c.stream_k || a.k / 128 < c.splits || lora)  // (the LoRA steps are 64 deep)
            rc = half_a ? launch_bn<128, 1, 8, 2, 2, 1, 64>(tmap, tmap_c, p, a.stream, pt, plb)
                        : launch_bn<128, 1, 8, 2, 2, 1>(tmap, tmap_c, p, a.stream, pt, plb);
        else
            rc = half_a ? launch_bn<128, 1, 8, 2, 2, 2, 64>(tmap, tmap_c, p, a.stream)
                        : launch_bn<128, 1, 8, 2, 2, 2>(tmap, tmap_c, p, a.stream);
    if (rc) return rc;
    if (c.splits > 1) {
        const size_t total4 = static_cast<size_t>(a.m) * a.n / 4;
        int blocks = static_cast<int>((total4 + 255) / 256);
        const int cap = device_sm_count() * 8;
        if (blocks > cap) blocks = cap;
        note_launch();
        rc = record_cuda_error(launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), a.stream, p.partial, p.C, p.S, a.m, a.n,
                                          c.splits, static_cast<int>(p.per_column)));
    }
    if (c.stream_k && p.m_tiles * p.n_tiles > plan.first_tile) {
        const int rem = p.m_tiles * p.n_tiles - plan.first_tile;
        const long long total = static_cast<long long>(rem) * p.k_iters;
        note_launch();
        rc = record_cuda_error(launch_pdl(streamk_fixup_kernel, dim3(rem, 16), dim3(256), a.stream, p.partial, p.C, p.S, a.m, a.n,
                                          p.m_tiles, p.k_iters, BM * c.mt, c.bn, plan.ctas, total, plan.first_tile,
                                          static_cast<int>(p.per_column)));
    }
    return rc;
}

}  // namespace kiln

// ---- the entry point that allocates nothing ---------------------------------------------------
//
// Some callers of this library cannot allocate device memory at call time and have no buffer to
// lend either: an inference server that hands every remaining byte of HBM to its KV-cache pool at
// start-up, or a serving loop that cannot afford the device-wide synchronisation a cudaMalloc or
// cudaFree implies.  For them the split-K scratch of the prefill kernel lives in a fixed array in
// the library's own device image.  Every GPU that loads the library holds these 16 MiB until the
// process exits.
namespace kiln {
namespace {

static __device__ __align__(256) float g_static_scratch[KILN_W4A16_NOALLOC_SCRATCH_BYTES / sizeof(float)];
static __device__ __align__(256) uint32_t g_static_status[64];

struct StaticDeviceState {
    float *scratch = nullptr;
    uint32_t *status = nullptr;
};

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the
// address has to be asked for, once per device, with that device current.
int static_state(StaticDeviceState **out) {
    static StaticDeviceState per_device[64];
    static std::mutex mu;
    int dev = 0;
    if (int rc = record_cuda_error(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= 64) return KILN_W4A16_ERR_ARG;
    std::lock_guard<std::mutex> lock(mu);
    StaticDeviceState &st = per_device[dev];
    if (!st.scratch) {
        void *p_scratch = nullptr, *p_status = nullptr;
        if (int rc = record_cuda_error(cudaGetSymbolAddress(&p_scratch, g_static_scratch))) return rc;
        if (int rc = record_cuda_error(cudaGetSymbolAddress(&p_status, g_static_status))) return rc;
        st.status = static_cast<uint32_t *>(p_status);
        st.scratch = static_cast<float *>(p_scratch);
    }
    *out = &st;
    return 0;
}

PrefillConfig noalloc_config(int m, int n, int k) {
    return choose_prefill(m, n, k, /*allow_pairs=*/false, /*allow_scratch=*/true, KILN_W4A16_NOALLOC_SCRATCH_BYTES);
}

}  // namespace

// Reads and clears the status word of the no-allocation entry's launches on the current device (0 if that entry has
// never run there).  No allocation: the word lives in the library image.
int static_status_read_clear(cudaStream_t st, uint32_t *out) {
    *out = 0;
    int dev = 0;
    if (int rc = record_cuda_error(cudaGetDevice(&dev))) return rc;
    if (dev < 0 || dev >= 64) return 0;
    StaticDeviceState *state = nullptr;
    if (int rc = static_state(&state)) return rc;
    if (int rc = record_cuda_error(cudaMemcpyAsync(out, state->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, st))) return rc;
    if (int rc = record_cuda_error(cudaStreamSynchronize(st))) return rc;
    if (*out != 0) {
        if (int rc = record_cuda_error(cudaMemsetAsync(state->status, 0, sizeof(uint32_t), st))) return rc;
        if (int rc = record_cuda_error(cudaStreamSynchronize(st))) return rc;
    }
    return 0;
}
}  // namespace kiln

extern "C" void kiln_w4a16_noalloc_plan(int m, int n, int k, int out[4]) {
    if (!out || m <= 0 || n <= 0 || k <= 0) return;
    const kiln::PrefillConfig c = kiln::noalloc_config(m, n, k);
    out[0] = c.bn;
    out[1] = c.splits;
    out[2] = c.mt;
    out[3] = c.stream_k;
}

extern "C" kiln_w4a16_status_t kiln_w4a16_gemm_bf16_noalloc(const void *A, const void *B, void *C, const void *s,
                                                            int m, int n, int k, int groupsize, void *stream) {
    using namespace kiln;
    if (m < 0 || n < 0 || k < 0) return KILN_W4A16_ERR_ARG;
    if (k % 128 != 0 || n % 256 != 0 || !(groupsize == -1 || groupsize == 128)) return KILN_W4A16_ERR_PROB_SHAPE;
    if (m == 0 || n == 0 || k == 0) return KILN_W4A16_OK;
    if (!A || !B || !C || !s) return KILN_W4A16_ERR_ARG;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C) |
         reinterpret_cast<uintptr_t>(s)) & 15)
        return KILN_W4A16_ERR_ALIGNMENT;
    if (!prefill_supported(m, n, k, groupsize)) return KILN_W4A16_ERR_KERN_SHAPE;

    // the best tiling whose split-K slabs fit the array (a tiling without a split always does); only a tiling forced
    // through the tuning hook can still ask for more
    const PrefillConfig c = noalloc_config(m, n, k);
    const size_t need = c.splits > 1 ? static_cast<size_t>(c.splits) * m * n * sizeof(float) : 0;
    if (need > KILN_W4A16_NOALLOC_SCRATCH_BYTES) return KILN_W4A16_ERR_STATIC_SCRATCH;

    StaticDeviceState *st = nullptr;
    if (int rc = static_state(&st)) return rc;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return KILN_W4A16_ERR_CUDA;

    CUtensorMap tmap;
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(m)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
    const cuuint32_t box[2] = {BK, BM};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(A), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return KILN_W4A16_ERR_CUDA;

    PrefillParams p{};
    p.B = static_cast<const uint4 *>(B);
    p.S = static_cast<const __half *>(s);
    p.C = static_cast<__nv_bfloat16 *>(C);
    // Nothing in the scratch has to start at zero: every split writes its whole [m, n] slab before the
    // reduction reads it, so what the previous call left behind is simply overwritten.
    p.partial = st->scratch;
    p.status = st->status;
    p.m = m;
    p.n = n;
    p.k = k;
    p.m_tiles = (m + BM - 1) / BM;
    p.n_tiles = n / c.bn;
    p.splits = c.splits;
    p.k_iters = k / BK;
    p.per_column = groupsize == -1;
    p.wait_limit_ns = g_wait_limit_ns;
    p.test_drop_a_load = -1;
    p.self_peer = -1;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    CUtensorMap tmap_c;
    if (!encode_c_map(enc, &tmap_c, C, m, n)) return KILN_W4A16_ERR_CUDA;
    int rc = c.bn == 256 ? launch_bn<256>(tmap, tmap_c, p, cs) : launch_bn<128>(tmap, tmap_c, p, cs);
    if (rc) return rc;
    if (c.splits > 1) {
        const size_t total4 = static_cast<size_t>(m) * n / 4;
        int blocks = static_cast<int>((total4 + 255) / 256);
        const int cap = device_sm_count() * 8;
        if (blocks > cap) blocks = cap;
        note_launch();
        rc = record_cuda_error(launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), cs, p.partial, p.C, p.S, m, n, c.splits,
                                          static_cast<int>(p.per_column)));
    }
    return rc;
}
