// Decode-shape W4A16 GEMM for sm_100a: C[m,n] = A[m,k] * dequant(B)[k,n], m small.
//
// Replaces the reference's `Marlin<256,1,8,8,4,8>` path
// (kiln-marlin-gemm/csrc/marlin_kernel.cu:197-700) with a different decomposition:
//
//  * HBM streaming, GEMV-like: the unit of work is one 4 KB run of the packed matrix
//    (one 64-column chunk x one 128-row scale group).  A warp reads a unit as eight
//    coalesced 512-byte loads (16 bytes per lane) that are all in flight at once, and keeps
//    a second unit in flight while it computes.
//  * in-register int4 -> bf16 dequant: `lop3` puts each nibble pair into the mantissa of
//    bf16x2 {128,128}; the "+128+8" offset is not subtracted per weight but removed once per
//    MMA tile by one extra MMA against a constant -136 fragment.
//  * bf16 m16n8k16 tensor-core MMAs with fp32 accumulation; the fp16 group scale is applied
//    once per 128-K group to the fp32 partial sums (exact scale, no bf16 rounding of it).
//  * split-K without global scratch: the K range is split over the warps of a CTA and over
//    the CTAs of a thread-block cluster; partial tiles meet in (distributed) shared memory
//    and are summed in a fixed order, so results are bit-reproducible.
//  * programmatic dependent launch: the first weight loads are issued before waiting for
//    the previous kernel in the stream, so back-to-back GEMMs overlap their ramp-up.
#include "w4a16_common.cuh"

namespace kiln {

struct DecodeParams {
    const __nv_bfloat16 *A;
    const uint4 *B;
    const __half *S;
    __nv_bfloat16 *C;
    int m, n, k;
    int groups;          // k / 128
    int groups_per_cta;  // K groups owned by one CTA of the cluster
    int pass_groups;     // K groups whose activations are staged in shared memory at a time
    int warps_n, warps_k;
    int per_column;      // groupsize == -1: one scale row, applied at the end
    int a_pitch;         // elements per staged activation row (pass_groups*128 + 8)
    int red_pitch;       // floats per reduction row (warps_n*64 + 8)
    int a_bytes;         // bytes of the activation stage
};

struct UnitRegs {
    uint4 w[8];
    uint4 sc[2];
};

__device__ __forceinline__ void load_unit(UnitRegs &u, const DecodeParams &p, int g, int chunk,
                                          int lane) {
    const int chunks = p.n >> 6;
    const uint4 *b = p.B + (static_cast<size_t>(g) * 8 * chunks + chunk) * 32 + lane;
#pragma unroll
    for (int kt = 0; kt < 8; ++kt) u.w[kt] = ld_stream_v4(b + static_cast<size_t>(kt) * chunks * 32);
    if (p.per_column) {
        u.sc[0] = make_uint4(0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u);  // fp16 ones
        u.sc[1] = u.sc[0];
    } else {
        // accumulator columns of this lane are chunk*64 + 8t + 2*(lane%4) + e; in the Marlin
        // scale order those sit at 16*(lane%4) + 8e + t: 32 contiguous bytes.
        const uint4 *s = reinterpret_cast<const uint4 *>(p.S + static_cast<size_t>(g) * p.n + chunk * 64 +
                                                         16 * (lane & 3));
        u.sc[0] = ld_stream_v4(s);
        u.sc[1] = ld_stream_v4(s + 1);
    }
}

__device__ __forceinline__ float half_at(const uint4 &v, int t) {
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
    const uint32_t w = words[t >> 1];
    return __half2float(__ushort_as_half(static_cast<unsigned short>((t & 1) ? (w >> 16) : (w & 0xFFFFu))));
}

template <int MT>
__device__ __forceinline__ void compute_unit(const UnitRegs &u, uint32_t a_addr, uint32_t a_mt_stride,
                                             float (&acc)[MT][8][4]) {
    float g[MT][8][4];
    float corr[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int i = 0; i < 4; ++i) corr[mt][i] = 0.f;
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) g[mt][t][i] = 0.f;
    }
#pragma unroll
    for (int kt = 0; kt < 8; ++kt) {
        uint32_t a[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) ldmatrix_x4(a[mt], a_addr + mt * a_mt_stride + kt * 32);
        const uint32_t xs[4] = {u.w[kt].x, u.w[kt].y, u.w[kt].z, u.w[kt].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t x = xs[j];
            const uint32_t p0 = lop3_and_or(x, kNibMask, kMagic128);
            const uint32_t p1 = lop3_and_or(x >> 4, kNibMask, kMagic128);
            const uint32_t p2 = lop3_and_or(x >> 8, kNibMask, kMagic128);
            const uint32_t p3 = lop3_and_or(x >> 12, kNibMask, kMagic128);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16_16816(g[mt][2 * j], a[mt], p0, p1);
                mma_bf16_16816(g[mt][2 * j + 1], a[mt], p2, p3);
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(corr[mt], a[mt], kNeg136x2, kNeg136x2);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        const float s0 = half_at(u.sc[0], t), s1 = half_at(u.sc[1], t);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            acc[mt][t][0] = fmaf(s0, g[mt][t][0] + corr[mt][0], acc[mt][t][0]);
            acc[mt][t][1] = fmaf(s1, g[mt][t][1] + corr[mt][1], acc[mt][t][1]);
            acc[mt][t][2] = fmaf(s0, g[mt][t][2] + corr[mt][2], acc[mt][t][2]);
            acc[mt][t][3] = fmaf(s1, g[mt][t][3] + corr[mt][3], acc[mt][t][3]);
        }
    }
}

// grid = (cluster_k, n / (64*warps_n), ceil(m / (16*MT))), cluster = (cluster_k, 1, 1),
// block = 32 * warps_n * warps_k.
template <int MT, bool PF>
__global__ void __launch_bounds__(MT == 1 ? 320 : 256) w4a16_decode_kernel(const DecodeParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __nv_bfloat16 *sA = reinterpret_cast<__nv_bfloat16 *>(smem);
    float *sRed = reinterpret_cast<float *>(smem + p.a_bytes);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wn = warp % p.warps_n, wk = warp / p.warps_n;
    const int chunk = blockIdx.y * p.warps_n + wn;
    const int m0 = blockIdx.z * (16 * MT);
    const int m_valid = min(16 * MT, p.m - m0);
    const uint32_t rank = cluster_ctarank(), csize = cluster_nctarank();

    const int gc0 = min(p.groups, static_cast<int>(rank) * p.groups_per_cta);
    const int gc1 = min(p.groups, gc0 + p.groups_per_cta);

    float acc[MT][8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int t = 0; t < 8; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[mt][t][i] = 0.f;

    // lane-constant part of the ldmatrix address: row (lane%8) + 8*((lane/8)%2), column 8*(lane/16)
    const uint32_t a_lane = smem_u32(sA) +
                            2u * (static_cast<uint32_t>((lane & 7) + ((lane >> 3) & 1) * 8) * p.a_pitch +
                                  static_cast<uint32_t>(lane >> 4) * 8);
    const uint32_t a_mt_stride = 2u * 16u * p.a_pitch;

    UnitRegs cur;
    bool first_pass = true;
    for (int pg0 = gc0; pg0 < gc1 || first_pass; pg0 += p.pass_groups) {
        const int pg1 = min(gc1, pg0 + p.pass_groups);
        const int plen = max(0, pg1 - pg0);
        const int gpw = (plen + p.warps_k - 1) / p.warps_k;
        const int g0 = min(pg1, pg0 + wk * gpw), g1 = min(pg1, g0 + gpw);

        // weights never depend on the previous kernel: get them moving first
        if (g0 < g1) load_unit(cur, p, g0, chunk, lane);
        if (first_pass) {
            pdl_launch_dependents();
            pdl_wait();
        } else {
            __syncthreads();  // everyone is done reading the previous pass' activations
        }
        // stage A[m0 .. m0+16MT, pg0*128 .. pg1*128) (zero rows past m)
        {
            const int vpr = plen * (kGroup / 8);  // 16-byte vectors per row
            const int total = 16 * MT * vpr;
            for (int v = tid; v < total; v += blockDim.x) {
                const int row = v / vpr, cv = v - row * vpr;
                uint4 val = make_uint4(0, 0, 0, 0);
                if (row < m_valid)
                    val = *reinterpret_cast<const uint4 *>(p.A + static_cast<size_t>(m0 + row) * p.k +
                                                           static_cast<size_t>(pg0) * kGroup + cv * 8);
                *reinterpret_cast<uint4 *>(sA + static_cast<size_t>(row) * p.a_pitch + cv * 8) = val;
            }
        }
        __syncthreads();

        for (int g = g0; g < g1; ++g) {
            const uint32_t a_addr = a_lane + 2u * static_cast<uint32_t>(g - pg0) * kGroup;
            if (PF) {
                UnitRegs nxt;
                const bool more = g + 1 < g1;
                if (more) load_unit(nxt, p, g + 1, chunk, lane);
                compute_unit<MT>(cur, a_addr, a_mt_stride, acc);
                if (more) cur = nxt;
            } else {
                compute_unit<MT>(cur, a_addr, a_mt_stride, acc);
                if (g + 1 < g1) load_unit(cur, p, g + 1, chunk, lane);
            }
        }
        first_pass = false;
    }

    // ---- reduction over the K-warps of the CTA, then over the CTAs of the cluster ----------
    {
        const int c = lane >> 2, qd = lane & 3;
        float *mine = sRed + static_cast<size_t>(wk) * (16 * MT) * p.red_pitch;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const int col = wn * 64 + 8 * t + 2 * qd;
                const int r0 = mt * 16 + c;
                if (r0 < m_valid)
                    *reinterpret_cast<float2 *>(mine + r0 * p.red_pitch + col) =
                        make_float2(acc[mt][t][0], acc[mt][t][1]);
                if (r0 + 8 < m_valid)
                    *reinterpret_cast<float2 *>(mine + (r0 + 8) * p.red_pitch + col) =
                        make_float2(acc[mt][t][2], acc[mt][t][3]);
            }
        }
    }
    __syncthreads();
    const int pairs_per_row = p.warps_n * 32;
    const int npairs = m_valid * pairs_per_row;
    if (p.warps_k > 1) {
        for (int idx = tid; idx < npairs; idx += blockDim.x) {
            const int row = idx / pairs_per_row, cp = idx - row * pairs_per_row;
            float *dst = sRed + row * p.red_pitch + 2 * cp;
            float2 s = *reinterpret_cast<float2 *>(dst);
            for (int w = 1; w < p.warps_k; ++w) {
                const float2 v =
                    *reinterpret_cast<float2 *>(dst + static_cast<size_t>(w) * (16 * MT) * p.red_pitch);
                s.x += v.x;
                s.y += v.y;
            }
            *reinterpret_cast<float2 *>(dst) = s;
        }
        __syncthreads();
    }
    if (csize > 1) cluster_sync_all();

    const int n0 = blockIdx.y * p.warps_n * 64;
    const int per_rank = (npairs + csize - 1) / csize;
    const int i0 = min(npairs, static_cast<int>(rank) * per_rank), i1 = min(npairs, i0 + per_rank);
    const uint32_t red_base = smem_u32(sRed);
    for (int idx = i0 + tid; idx < i1; idx += blockDim.x) {
        const int row = idx / pairs_per_row, cp = idx - row * pairs_per_row;
        const uint32_t off = red_base + 4u * static_cast<uint32_t>(row * p.red_pitch + 2 * cp);
        float2 s;
        if (csize > 1) {
            s = make_float2(0.f, 0.f);
            for (uint32_t r = 0; r < csize; ++r) {
                const float2 v = ld_dsmem_f2(map_to_cta(off, r));
                s.x += v.x;
                s.y += v.y;
            }
        } else {
            s = *reinterpret_cast<const float2 *>(sRed + row * p.red_pitch + 2 * cp);
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
    // keep this CTA's shared memory alive until every peer has read it
    if (csize > 1) cluster_sync_all();
}

// ---- host: decomposition heuristic and launch ---------------------------------------------

namespace {

constexpr int kPassCapMt1 = 10;  // groups of A staged at once (16 rows): 10*128*16*2 B = 40 KB
constexpr int kPassCapMt2 = 5;

struct DecodeConfig {
    int mt, cluster_k, warps_k, warps_n, groups_per_cta, pass_groups;
    bool prefetch;
};

int ceil_div(int a, int b) { return (a + b - 1) / b; }

DecodeConfig choose_config(int m, int n, int k, const DecodeOverride &ov) {
    DecodeConfig c{};
    const int groups = k / kGroup, chunks = n / kChunkCols;
    c.mt = m <= 16 ? 1 : 2;
    c.prefetch = c.mt == 1;
    const int mblocks = ceil_div(m, 16 * c.mt);
    const int sms = device_sm_count();
    const int max_warps = c.mt == 1 ? 10 : 8;

    int wn = m <= 4 ? 1 : (m <= 8 ? 2 : 4);
    int ck, wk;
    if (ov.cluster_k > 0 && ov.warps_k > 0 && ov.warps_n > 0) {
        ck = ov.cluster_k;
        wk = ov.warps_k;
        wn = ov.warps_n;
    } else {
        // aim for about one resident wave: SMs x 12 warps (MT=1) or x 8 (MT=2)
        const long long capacity = static_cast<long long>(sms) * (c.mt == 1 ? 12 : 8);
        const long long units = static_cast<long long>(groups) * chunks * mblocks;
        const int upw = static_cast<int>(units / capacity > 0 ? (units + capacity - 1) / capacity : 1);
        const int kwarps = ceil_div(groups, upw);  // K-warps wanted per 64-column chunk
        const int wk_cap = max_warps / wn > 0 ? max_warps / wn : 1;
        ck = 1;
        while (ck < 8 && ceil_div(kwarps, ck) > wk_cap) ck *= 2;
        wk = ceil_div(kwarps, ck);
        if (wk > wk_cap) wk = wk_cap;
        if (wk < 1) wk = 1;
    }
    while (chunks % wn) wn /= 2;
    if (ck > 8) ck = 8;
    if (ck > groups) ck = 1;
    c.cluster_k = ck;
    c.warps_k = wk;
    c.warps_n = wn;
    c.groups_per_cta = ceil_div(groups, ck);
    const int cap = c.mt == 1 ? kPassCapMt1 : kPassCapMt2;
    c.pass_groups = c.groups_per_cta < cap ? c.groups_per_cta : cap;
    return c;
}

template <int MT, bool PF>
int launch_one(const DecodeParams &p, const DecodeConfig &c, int m, cudaStream_t stream) {
    static bool attr_set[64] = {};
    const size_t smem = static_cast<size_t>(p.a_bytes) +
                        sizeof(float) * static_cast<size_t>(c.warps_k) * 16 * MT * p.red_pitch;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 64 && !attr_set[dev]) {
        if (int rc = record_cuda_error(cudaFuncSetAttribute(w4a16_decode_kernel<MT, PF>,
                                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                            160 * 1024)))
            return rc;
        attr_set[dev] = true;
    }
    if (smem > 160 * 1024) return KILN_W4A16_ERR_KERN_SHAPE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(c.cluster_k, p.n / (kChunkCols * c.warps_n), (m + 16 * MT - 1) / (16 * MT));
    cfg.blockDim = dim3(32 * c.warps_n * c.warps_k);
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
    return record_cuda_error(cudaLaunchKernelEx(&cfg, w4a16_decode_kernel<MT, PF>, p));
}

}  // namespace

int launch_decode_regs(const GemmArgs &a, const DecodeOverride &ov) {
    const DecodeConfig c = choose_config(a.m, a.n, a.k, ov);
    if (c.warps_n * c.warps_k * 32 > (c.mt == 1 ? 320 : 256)) return KILN_W4A16_ERR_KERN_SHAPE;
    DecodeParams p{};
    p.A = static_cast<const __nv_bfloat16 *>(a.A);
    p.B = static_cast<const uint4 *>(a.B);
    p.S = static_cast<const __half *>(a.S);
    p.C = static_cast<__nv_bfloat16 *>(a.C);
    p.m = a.m;
    p.n = a.n;
    p.k = a.k;
    p.groups = a.k / kGroup;
    p.groups_per_cta = c.groups_per_cta;
    p.pass_groups = c.pass_groups;
    p.warps_n = c.warps_n;
    p.warps_k = c.warps_k;
    p.per_column = a.groupsize == -1;
    p.a_pitch = c.pass_groups * kGroup + 8;
    p.red_pitch = c.warps_n * 64 + 8;
    p.a_bytes = 16 * c.mt * p.a_pitch * 2;
    if (c.mt == 1) return launch_one<1, true>(p, c, a.m, a.stream);
    return launch_one<2, false>(p, c, a.m, a.stream);
}

}  // namespace kiln
