// Decode-shape W4A16 GEMM for sm_100a: C[m,n] = A[m,k] * dequant(B)[k,n], m small.
//
// Replaces the reference's `Marlin<256,1,8,8,4,8>` path
// (kiln-marlin-gemm/csrc/marlin_kernel.cu:197-700) with a different decomposition:
//
//  * HBM streaming, GEMV-like.  The unit of work is one "stage": one 128-row scale group of
//    WN adjacent 64-column chunks = 8 runs of WN*512 contiguous bytes of the packed matrix
//    plus WN*128 bytes of scales.  A producer warp moves stages global -> shared with bulk
//    asynchronous copies (TMA, mbarrier completion) into a ring, so the bytes in flight per SM
//    are set by the ring depth, not by registers or by how many warps are resident, and the
//    weight stream starts before the previous kernel in the stream has finished
//    (programmatic dependent launch; only the activations, which the consumer warps stage
//    themselves with plain loads, wait for it).
//  * consumer warps: in-register int4 -> bf16 dequant (`lop3` puts each nibble pair into the
//    mantissa of bf16x2 {128,128}); the +128+8 offset is not
//    subtracted per weight but removed per MMA tile by one extra MMA against a constant
//    -136 fragment; bf16 m16n8k16 tensor-core MMAs with fp32 accumulation; the fp16 group
//    scale is applied once per 128-K group to the fp32 partial sums (exact scale).
//  * split-K without global scratch: K is split over teams of warps inside a CTA and over
//    the CTAs of a thread-block cluster; partial tiles meet in (distributed) shared memory
//    and are summed in a fixed order, so results are bit-reproducible.
//  * every wait on an mbarrier is bounded (see w4a16_async.cuh).
#include "w4a16_async.cuh"

namespace kiln {
namespace {

struct DecodeParams {
    const __nv_bfloat16 *A;
    const uint8_t *B;  // packed weights, byte view
    const __half *S;
    __nv_bfloat16 *C;
    uint32_t *status;
    int m, n, k;
    int groups;          // k / 128
    int groups_per_cta;  // K groups owned by one CTA of the cluster
    int warps_n, warps_k;
    int stages;          // ring depth
    int window;          // stages kept in flight by the producer
    int per_column;      // groupsize == -1: one scale row, applied at the end
    int a_pitch;         // bytes per staged activation row (groups_per_cta*256 + 16)
    int red_pitch;       // floats per reduction row (warps_n*64 + 8)
    // shared-memory carve-up (bytes from the 128-byte aligned base)
    int off_ring, off_red, off_recv, off_bar, stage_bytes;
};

__device__ __forceinline__ float half_bits_to_float(uint32_t w, int hi) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(hi ? (w >> 16) : (w & 0xFFFFu))));
}

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Nibble alignment shift.  Measured on B200: plain ALU shifts beat high multiplies on the FMA pipe here
// (gate+up M=1 11.6 us vs 12.7 us; IMAD.HI issues at a quarter of the rate), so the shifts stay on the ALU.
template <int S>
__device__ __forceinline__ uint32_t shr_mul(uint32_t x) {
    return x >> S;
}

// One stage for one warp: 8 K-tiles of one 64-column chunk.
//
// The MMA is issued transposed: the weights are its 16x16 "A" operand (16 output columns x 16 K)
// and the activations its 16x8 "B" operand (16 K x 8 batch rows).  A packed word is exactly
// one such A fragment -- nibble pairs (0,4) (2,6) (1,5) (3,7) are a0..a3 -- so a batch of up to 8
// rows costs one MMA per word instead of two, and the accumulators D^T[16 cols x 8 rows] of a
// lane sit on columns c + 8t, whose eight scales are one 16-byte run of the Marlin scale order.
template <int NB>
__device__ __forceinline__ void compute_stage(uint32_t w_addr, uint32_t w_kt_stride, uint32_t s_addr, bool scaled,
                                              uint32_t a_addr, float (&acc)[4][NB][4]) {
    float g[4][NB][4];
    float corr[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) corr[nb][i] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) g[j][nb][i] = 0.f;
    }
    uint4 sc = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);  // fp16 ones
    if (scaled) sc = lds_v4(s_addr);
    const uint32_t neg[4] = {kNeg136x2, kNeg136x2, kNeg136x2, kNeg136x2};
#pragma unroll
    for (int kt = 0; kt < 8; ++kt) {
        const uint4 w = lds_v4(w_addr + kt * w_kt_stride);
        uint32_t b[NB][2];
        if (NB == 1) {
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
                         : "=r"(b[0][0]), "=r"(b[0][1])
                         : "r"(a_addr + kt * 32));
        } else {
            uint32_t r[4];
            ldmatrix_x4(r, a_addr + kt * 32);
            b[0][0] = r[0];
            b[0][1] = r[1];
            b[NB - 1][0] = r[2];
            b[NB - 1][1] = r[3];
        }
        const uint32_t xs[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = xs[j];
            uint32_t f[4];
            f[0] = lop3_and_or(x, kNibMask, kMagic128);              // col c,   K 2qd, 2qd+1
            f[2] = lop3_and_or(shr_mul<4>(x), kNibMask, kMagic128);   // col c,   K 2qd+8, 2qd+9
            f[1] = lop3_and_or(shr_mul<8>(x), kNibMask, kMagic128);   // col c+8, K 2qd, 2qd+1
            f[3] = lop3_and_or(shr_mul<12>(x), kNibMask, kMagic128);  // col c+8, K 2qd+8, 2qd+9
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) mma_bf16_16816(g[j][nb], f, b[nb][0], b[nb][1]);
        }
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_bf16_16816(corr[nb], neg, b[nb][0], b[nb][1]);
    }
    const uint32_t sw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float s0 = half_bits_to_float(sw[j], 0), s1 = half_bits_to_float(sw[j], 1);  // cols 16j+c, 16j+c+8
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            acc[j][nb][0] = fmaf(s0, g[j][nb][0] + corr[nb][0], acc[j][nb][0]);
            acc[j][nb][1] = fmaf(s0, g[j][nb][1] + corr[nb][1], acc[j][nb][1]);
            acc[j][nb][2] = fmaf(s1, g[j][nb][2] + corr[nb][0], acc[j][nb][2]);
            acc[j][nb][3] = fmaf(s1, g[j][nb][3] + corr[nb][1], acc[j][nb][3]);
        }
    }
}

// grid = (cluster_k, n / (64*warps_n), ceil(m / (8*NB))), cluster = (cluster_k, 1, 1),
// block = 32 * (1 + warps_n * warps_k): warp 0 produces, warp 1 + wk*warps_n + wn consumes
// chunk wn of the stages i with i % warps_k == wk.
template <int NB>
__global__ void __launch_bounds__(288, NB == 1 ? 2 : 1) w4a16_decode_kernel(const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    uint8_t *base_gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t sA = base, sRing = base + p.off_ring, sBar = base + p.off_bar;
    float *sRed = reinterpret_cast<float *>(base_gen + p.off_red);
    auto full = [&](int s) { return sBar + 8u * s; };
    auto empty = [&](int s) { return sBar + 8u * (p.stages + s); };
    volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(base_gen + p.off_bar + 8 * (2 * p.stages + 1));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int kRows = 8 * NB;
    const int m0 = blockIdx.z * kRows;
    const int m_valid = min(kRows, p.m - m0);
    const int chunk0 = blockIdx.y * p.warps_n;
    const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();
    const int gc0 = min(p.groups, static_cast<int>(rank) * p.groups_per_cta);
    const int gc1 = min(p.groups, gc0 + p.groups_per_cta);
    const int nst = gc1 - gc0;  // stages this CTA streams

    if (tid < p.stages) {  // one thread per ring slot (a loop in one thread cost ~0.3 us of every launch)
        mbar_init(full(tid), 1);
        mbar_init(empty(tid), p.warps_n);
        if (tid == 0) *abort_flag = 0;
        mbar_init_fence();
    }
    __syncthreads();
    pdl_launch_dependents();

    const int nwarps_c = p.warps_n * p.warps_k;
    float acc[4][NB][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[j][nb][i] = 0.f;

    if (warp == 0) {
        // ---------------- producer ----------------
        const uint32_t w_row_bytes = static_cast<uint32_t>(p.warps_n) * 512u;
        const uint32_t s_bytes = p.per_column ? 0u : static_cast<uint32_t>(p.warps_n) * 128u;
        const uint32_t tx = 8u * w_row_bytes + s_bytes;
        const size_t b_row_pitch = static_cast<size_t>(p.n) * 8;  // bytes per packed row (16 K)
        bool ok = true;
        auto issue_stage = [&](int i) {
            const int s = i % p.stages;
            const int g = gc0 + i;
            const uint32_t dst = sRing + s * p.stage_bytes;
            if (lane == 0) mbar_arrive_expect_tx(full(s), tx);
            __syncwarp();
            if (lane < 8)
                bulk_g2s(dst + lane * w_row_bytes,
                         p.B + (static_cast<size_t>(g) * 8 + lane) * b_row_pitch + static_cast<size_t>(chunk0) * 512,
                         w_row_bytes, full(s));
            else if (lane == 8 && s_bytes)
                bulk_g2s(dst + 8 * w_row_bytes, p.S + static_cast<size_t>(g) * p.n + chunk0 * 64, s_bytes, full(s));
        };
        // Weights never depend on the previous kernel: start them before waiting for it.  Only `window`
        // stages are kept in flight per CTA: requesting everything at once makes the memory system serve all
        // copies side by side, so that the first stage lands about as late as the last (measured: first
        // data after 4.2 us instead of ~1.3 us) and the consumers start late.
        const int window = min(p.window, p.stages);
        const int pre = min(nst, window);
        for (int i = 0; i < pre; ++i) issue_stage(i);
        for (int i = pre; i < nst && ok; ++i) {
            const int j = i - window;  // this stage must have landed before stage i is requested
            ok = mbar_wait(full(j % p.stages), (j / p.stages) & 1, abort_flag, p.status, 0x1000u | (j % p.stages));
            if (ok && i >= p.stages) {  // slot reuse: its previous contents must have been consumed
                const int s = i % p.stages;
                ok = mbar_wait(empty(s), ((i / p.stages) & 1) ^ 1, abort_flag, p.status, 0x1100u | s);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (ok) issue_stage(i);
        }
        if (!ok && lane == 0) {
            // drain what was issued before leaving (shared memory must outlive the copies)
            for (int i = max(0, nst - p.stages); i < nst; ++i) mbar_wait_quiet(full(i % p.stages), (i / p.stages) & 1);
        }
    } else if (warp <= nwarps_c) {
        // ---------------- consumers ----------------
        const int cw = warp - 1;
        const int wn = cw % p.warps_n, wk = cw / p.warps_n;
        const int qd = lane & 3, c = lane >> 2;
        // lane-constant part of the ldmatrix address.  x2: lanes 0-7 rows 0-7 at K+0, lanes 8-15 the same
        // rows at K+8.  x4 adds rows 8-15 for lanes 16-31.
        // Only the valid rows are staged: rows past m read the last valid row again (their products land in
        // accumulator rows that are never stored).
        const int a_row = min((lane & 7) + (NB == 2 ? (lane >> 4) * 8 : 0), m_valid - 1);
        const uint32_t a_lane = sA + static_cast<uint32_t>(a_row) * p.a_pitch + static_cast<uint32_t>((lane >> 3) & 1) * 16u;
        const uint32_t w_kt_stride = static_cast<uint32_t>(p.warps_n) * 512u;
        bool ok = true;
        // Activations: staged by the consumer warps themselves with plain loads (they come from L2), not by a
        // bulk copy of the producer: a copy queued behind the weight stages in flight landed last (2.4-4.2 us
        // after the launch) and held every consumer back.  Only this depends on the previous kernel.
        pdl_wait();
        {
            const int vec_per_row = nst * 16;  // 16-byte pieces per row in this CTA's K range
            const int ctid = tid - 32;
            for (int idx = ctid; idx < m_valid * vec_per_row; idx += nwarps_c * 32) {
                const int r = idx / vec_per_row, v = idx - r * vec_per_row;
                const uint4 val = ld_cg_v4(reinterpret_cast<const uint4 *>(
                    p.A + static_cast<size_t>(m0 + r) * p.k + static_cast<size_t>(gc0) * kGroup + v * 8));
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(sA + r * p.a_pitch + v * 16), "r"(val.x),
                             "r"(val.y), "r"(val.z), "r"(val.w)
                             : "memory");
            }
            asm volatile("bar.sync 1, %0;" ::"r"(nwarps_c * 32) : "memory");
        }
        for (int i = wk; i < nst && ok; i += p.warps_k) {
            const int s = i % p.stages;
            const uint32_t ph = (i / p.stages) & 1;
            if (!(ok = mbar_wait(full(s), ph, abort_flag, p.status, 0x1300u | s))) break;
            const uint32_t st = sRing + s * p.stage_bytes;
            compute_stage<NB>(st + wn * 512u + lane * 16u, w_kt_stride, st + 8u * w_kt_stride + wn * 128u + 16u * c,
                              !p.per_column, a_lane + static_cast<uint32_t>(i) * 256u, acc);
            __syncwarp();
            if (lane == 0 && nst > p.stages) mbar_arrive(empty(s));  // only a reused slot needs the release
        }
        // this warp's partial tile -> shared memory: acc[j][nb][i] is column 16j + c + 8*(i/2) of the chunk,
        // batch row 8nb + 2qd + (i%2)
        float *mine = sRed + static_cast<size_t>(wk) * kRows * p.red_pitch;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = 8 * nb + 2 * qd + (i & 1);
                    if (row < m_valid) mine[row * p.red_pitch + wn * 64 + 16 * j + c + 8 * (i >> 1)] = acc[j][nb][i];
                }
    }
    __syncthreads();

    // ---- reduction over the K-teams of the CTA, then over the CTAs of the cluster -----------
    // Output pairs (two adjacent columns) are dealt to the cluster ranks in contiguous slices.  Every CTA
    // sums its K-teams and pushes each pair into the owning rank's receive buffer, slot [sender rank];
    // after ONE cluster barrier the owner adds the slots in rank order and writes C.  Nobody touches a
    // peer's shared memory after that barrier, so CTAs may exit without a second one.
    const int pairs_per_row = p.warps_n * 32;
    const int npairs = m_valid * pairs_per_row;
    const int per_rank = (npairs + csize - 1) / csize;
    const uint32_t recv_base = base + p.off_recv;
    float2 *recv = reinterpret_cast<float2 *>(base_gen + p.off_recv);
    for (int idx = tid; idx < npairs; idx += blockDim.x) {
        const int row = idx / pairs_per_row, cp = idx - row * pairs_per_row;
        const float *src = sRed + row * p.red_pitch + 2 * cp;
        float2 s = *reinterpret_cast<const float2 *>(src);
        for (int w = 1; w < p.warps_k; ++w) {
            const float2 v = *reinterpret_cast<const float2 *>(src + static_cast<size_t>(w) * kRows * p.red_pitch);
            s.x += v.x;
            s.y += v.y;
        }
        if (csize > 1) {
            const int owner = idx / per_rank, j = idx - owner * per_rank;
            st_dsmem_f2(map_to_cta(recv_base + 8u * static_cast<uint32_t>(rank * per_rank + j), owner), s);
        } else {
            recv[idx] = s;
        }
    }
    if (csize > 1)
        cluster_sync_all();
    else
        __syncthreads();
    pdl_wait();  // every thread that writes C orders itself after the previous kernel
    const int n0 = chunk0 * 64;
    const int i0 = min(npairs, static_cast<int>(rank) * per_rank), i1 = min(npairs, i0 + per_rank);
    for (int idx = i0 + tid; idx < i1; idx += blockDim.x) {
        const int row = idx / pairs_per_row, cp = idx - row * pairs_per_row;
        float2 s = recv[idx - i0];
        for (uint32_t r = 1; r < csize; ++r) {
            const float2 v = recv[r * per_rank + (idx - i0)];
            s.x += v.x;
            s.y += v.y;
        }
        const int col = n0 + 2 * cp;
        if (p.per_column) {
            const int pos = scale_single_pos(col);  // col is even: col+1 sits at pos+1
            s.x *= __half2float(p.S[pos]);
            s.y *= __half2float(p.S[pos + 1]);
        }
        *reinterpret_cast<__nv_bfloat162 *>(p.C + static_cast<size_t>(m0 + row) * p.n + col) =
            __floats2bfloat162_rn(s.x, s.y);
    }
}

// ---- host: decomposition heuristic and launch ---------------------------------------------

struct DecodeConfig {
    int nb, cluster_k, warps_k, warps_n, groups_per_cta, stages;
};

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Shared memory one CTA may use so that two CTAs (16 consumer warps) stay resident per SM.
constexpr int kSmemBudget = 108 * 1024;

int a_stage_bytes(int rows, int groups_per_cta) { return rows * (groups_per_cta * 256 + 16); }
int red_bytes(int nb, int wk, int wn) { return 4 * wk * 8 * nb * (wn * 64 + 8) + 8 * (8 * nb * wn * 32 + 8) + 128; }

DecodeConfig choose_config(int m, int n, int k, const DecodeOverride &ov) {
    DecodeConfig c{};
    const int groups = k / kGroup, chunks = n / kChunkCols;
    c.nb = m <= 8 ? 1 : 2;
    const int mblocks = ceil_div(m, 8 * c.nb);
    const int sms = device_sm_count();
    int wn = 1, ck = 1, wk = 8;
    if (ov.cluster_k > 0 && ov.warps_k > 0 && ov.warps_n > 0) {
        ck = ov.cluster_k;
        wk = ov.warps_k;
        wn = ov.warps_n;
    } else {
        // Rule fitted to sweeps over (cluster_k, warps_k, warps_n) on the Qwen3.5-4B projection shapes:
        // two chunks per CTA (1 KB bulk copies, activations shared by two warps), the smallest cluster
        // split that gives at least one CTA per SM while every CTA keeps two or more K groups, and
        // four K-teams (two when a batch needs two MMAs per word and the registers that go with it, or when
        // a CTA streams eight or more groups: two long-running teams then beat four short ones).
        wn = chunks % 2 == 0 ? 2 : 1;
        ck = 1;
        while (ck < 8 && static_cast<long long>(chunks / wn) * mblocks * ck < sms && groups / (ck * 2) >= 2) ck *= 2;
        int gpc = ceil_div(groups, ck);
        wk = (c.nb == 1 && gpc < 8) ? 4 : 2;
        if (wk > gpc) wk = gpc;
        // A projection so narrow that even the widest cluster split leaves most SMs idle (k, v: 512 columns):
        // one chunk per CTA doubles the CTAs, and eight warps (whatever the number of K groups) shorten the
        // activation staging and the reduction, which dominate such a launch.
        if (static_cast<long long>(chunks / wn) * mblocks * 8 < sms / 2) {
            wn = 1;
            ck = 8;
            while (ck > 1 && groups / ck < 2) ck /= 2;
            wk = 8;
        }
        // Measured exceptions (B200, CUDA-graph replay over rotating weights), keyed by the shape:
        struct Tuned {
            int k, n, nb, ck, wk, wn;
        };
        static const Tuned kTuned[] = {
            {2560, 4096, 1, 8, 4, 1},   // q:      5.17 us at M=8 (rule: 5.44)
            {2560, 4096, 2, 4, 4, 2},   // q:      6.31 us at M=16 (rule: 8.40)
            {2560, 8192, 1, 4, 3, 2},   // GDN-in: 5.61 us at M=1 (rule: 6.37)
        };
        for (const Tuned &t : kTuned)
            if (t.k == k && t.n == n && t.nb == c.nb) {
                ck = t.ck;
                wk = t.wk;
                wn = t.wn;
            }
    }
    while (chunks % wn) wn /= 2;
    if (ck > 8) ck = 8;
    while (ck > groups) ck /= 2;
    c.cluster_k = ck;
    c.warps_k = wk;
    c.warps_n = wn;
    c.groups_per_cta = ceil_div(groups, ck);
    // Ring depth: whatever the per-CTA budget leaves.  When the CTA streams more stages than the ring
    // holds, slots are reused, and then every slot must belong to exactly one K-team (depth a multiple
    // of warps_k): a team that skipped a fill of a slot could not tell fills apart by barrier parity.
    const int stage_bytes = wn * (8 * 512 + 128);
    const int rows = m < 8 * c.nb ? m : 8 * c.nb;  // activation rows a CTA stages
    const int room = kSmemBudget - a_stage_bytes(rows, c.groups_per_cta) - red_bytes(c.nb, wk, wn) - 512;
    int max_stages = room / stage_bytes;
    if (max_stages > 16) max_stages = 16;
    if (max_stages < 1) max_stages = 1;
    if (c.groups_per_cta <= max_stages) {
        c.stages = c.groups_per_cta;
    } else {
        if (wk > max_stages) wk = max_stages;
        c.warps_k = wk;
        c.stages = (max_stages / wk) * wk;
    }
    return c;
}

template <int NB>
int launch_one(DecodeParams &p, const DecodeConfig &c, int m, cudaStream_t stream) {
    static bool attr_set[64] = {};
    constexpr int kMaxSmem = 200 * 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        if (int rc = record_cuda_error(
                cudaFuncSetAttribute(w4a16_decode_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem)))
            return rc;
        attr_set[dev] = true;
    }
    // carve-up: [A rows][ring][reduction tiles][barriers]
    auto align = [](int x, int a) { return (x + a - 1) / a * a; };
    p.a_pitch = c.groups_per_cta * 256 + 16;
    p.stage_bytes = c.warps_n * (8 * 512 + 128);
    p.red_pitch = c.warps_n * 64 + 8;
    p.off_ring = align((m < 8 * NB ? m : 8 * NB) * p.a_pitch, 128);
    p.off_red = p.off_ring + align(c.stages * p.stage_bytes, 128);
    p.off_recv = p.off_red + align(static_cast<int>(sizeof(float)) * c.warps_k * 8 * NB * p.red_pitch, 128);
    p.off_bar = p.off_recv + align(8 * (8 * NB * c.warps_n * 32 + c.cluster_k), 128);
    const size_t smem = static_cast<size_t>(p.off_bar) + 8 * (2 * c.stages + 2) + 128;
    if (smem > kMaxSmem) return KILN_W4A16_ERR_KERN_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(c.cluster_k, p.n / (kChunkCols * c.warps_n), (m + 8 * NB - 1) / (8 * NB));
    cfg.blockDim = dim3(32 * (1 + c.warps_n * c.warps_k));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = c.cluster_k;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 2;
    if (cfg.gridDim.y > 65535 || cfg.gridDim.z > 65535) return KILN_W4A16_ERR_KERN_SHAPE;
    note_launch();
    return record_cuda_error(cudaLaunchKernelEx(&cfg, w4a16_decode_kernel<NB>, p));
}

}  // namespace

int launch_decode(const GemmArgs &a, const DecodeOverride &ov) {
    if (ov.cluster_k < 0) {  // A/B hook: the register-prefetch variant
        DecodeOverride o2{-ov.cluster_k, ov.warps_k, ov.warps_n};
        return launch_decode_regs(a, o2);
    }
    uint32_t *status = device_status_word();
    if (!status) return KILN_W4A16_ERR_CUDA;
    const DecodeConfig c = choose_config(a.m, a.n, a.k, ov);
    if ((1 + c.warps_n * c.warps_k) * 32 > 288) return KILN_W4A16_ERR_KERN_SHAPE;
    if (c.stages < 1 || (c.groups_per_cta > c.stages && c.stages % c.warps_k != 0)) return KILN_W4A16_ERR_KERN_SHAPE;
    // a CTA's K range must fit the activation stage: fall back to more cluster ranks is not possible
    // past 8, so very long K runs go through the register variant, which stages K in passes
    if ((a.m < 8 * c.nb ? a.m : 8 * c.nb) * (c.groups_per_cta * 256 + 16) > 96 * 1024)
        return launch_decode_regs(a, DecodeOverride{0, 0, 0});
    DecodeParams p{};
    p.A = static_cast<const __nv_bfloat16 *>(a.A);
    p.B = static_cast<const uint8_t *>(a.B);
    p.S = static_cast<const __half *>(a.S);
    p.C = static_cast<__nv_bfloat16 *>(a.C);
    p.status = status;
    p.m = a.m;
    p.n = a.n;
    p.k = a.k;
    p.groups = a.k / kGroup;
    p.groups_per_cta = c.groups_per_cta;
    p.warps_n = c.warps_n;
    p.warps_k = c.warps_k;
    p.stages = c.stages;
    p.window = 8;  // swept 2..16 on B200: 8 is best by a few percent (gate+up M=1: 10.3 us vs 10.8 at 4)
    p.per_column = a.groupsize == -1;
    if (c.nb == 1) return launch_one<1>(p, c, a.m, a.stream);
    return launch_one<2>(p, c, a.m, a.stream);
}

}  // namespace kiln
