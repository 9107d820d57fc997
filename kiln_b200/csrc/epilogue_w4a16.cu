// Small kernels around the W4A16 GEMM's epilogue options.
//
//  * lora_down_kernel: t = scale * x * A^T, the rank-r projection of kiln's LoRA delta
//    (kiln-model/src/lora_loader.rs:213-233: delta = x @ A^T @ B^T * scale).  The GEMM kernel then adds t * B^T to its
//    fp32 sums before rounding, so the delta never exists as a matrix of its own.
//  * finish_kernel: for batch sizes beyond the decode kernel's range, where the options are not fused yet:
//    C = epilogue(base), base being the bf16 GEMM result in the workspace (LoRA delta added, SwiGLU applied).
#include "w4a16_common.cuh"

namespace kiln {
namespace {

// grid = (ceil(r / 8), m), block = 256: warp w of a CTA computes t[row][8 * blockIdx.x + w].
// (bf16_out: t is a bf16 [m, r] matrix, the form the tcgen05 kernel reads as an operand tile)
__device__ __forceinline__ void store_t(void *t, size_t idx, float v, int bf16_out) {
    if (bf16_out)
        static_cast<__nv_bfloat16 *>(t)[idx] = __float2bfloat16(v);
    else
        static_cast<float *>(t)[idx] = v;
}

__global__ void __launch_bounds__(256) lora_down_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a,
                                                        float scale, int k, int r, void *__restrict__ t, int bf16_out) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.y, j = blockIdx.x * 8 + warp;
    pdl_wait();  // x may be the previous kernel's output; t may still be read by it
    if (j >= r) return;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(row) * k);
    const uint4 *ar = reinterpret_cast<const uint4 *>(a + static_cast<size_t>(j) * k);
    float sum = 0.f;
    for (int i = lane; i < k / 8; i += 32) {
        const uint4 xv = ld_cg_v4(xr + i), av = ar[i];
        const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w}, as[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
            sum += __uint_as_float(xs[e] << 16) * __uint_as_float(as[e] << 16) +
                   __uint_as_float(xs[e] & 0xFFFF0000u) * __uint_as_float(as[e] & 0xFFFF0000u);
    }
#pragma unroll
    for (int sh = 16; sh >= 1; sh >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sh);
    if (lane == 0) store_t(t, static_cast<size_t>(row) * r + j, sum * scale, bf16_out);
}

// The same for larger batches: a CTA takes eight rows of x, so that every adapter row it reads serves eight dot products
// (the kernel above re-reads the whole adapter once per row of x), and two adapter rows, each split over four warps along
// K (the sums meet in shared memory): enough CTAs to fill the GPU at continuous-batching sizes and a four times shorter
// loop per warp.  grid = (ceil(r / 2), ceil(m / 8)), block = 256.
__global__ void __launch_bounds__(256) lora_down_rows8_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ a,
                                                              float scale, int m, int k, int r, void *__restrict__ t, int bf16_out) {
    __shared__ float part[8][8];  // [warp][row of x]
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row0 = blockIdx.y * 8, j = blockIdx.x * 2 + (warp >> 2), kq = warp & 3;
    pdl_wait();  // x may be the previous kernel's output; t may still be read by it
    float sum[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (j < r) {
        const uint4 *ar = reinterpret_cast<const uint4 *>(a + static_cast<size_t>(j) * k);
        const int pieces = k / 8, per = (pieces + 3) / 4;  // 16-byte pieces of a row, and of this warp's quarter of K
        const int i1 = min(pieces, (kq + 1) * per);
        for (int i = kq * per + lane; i < i1; i += 32) {
            const uint4 av = ar[i];
            const uint32_t as[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                const int row = row0 + rr < m ? row0 + rr : m - 1;  // (rows past m repeat the last one; their sums are dropped)
                const uint4 xv = ld_cg_v4(reinterpret_cast<const uint4 *>(x + static_cast<size_t>(row) * k) + i);
                const uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    sum[rr] += __uint_as_float(xs[e] << 16) * __uint_as_float(as[e] << 16) +
                               __uint_as_float(xs[e] & 0xFFFF0000u) * __uint_as_float(as[e] & 0xFFFF0000u);
            }
        }
    }
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) {
        float v = sum[rr];
#pragma unroll
        for (int sh = 16; sh >= 1; sh >>= 1) v += __shfl_xor_sync(0xffffffffu, v, sh);
        if (lane == 0) part[warp][rr] = v;
    }
    __syncthreads();
    if (threadIdx.x < 16) {  // the CTA's 2 x 8 results: the four K quarters are added in a fixed order
        const int jj = threadIdx.x >> 3, rr = threadIdx.x & 7, jo = blockIdx.x * 2 + jj;
        const float v = (part[4 * jj][rr] + part[4 * jj + 1][rr]) + (part[4 * jj + 2][rr] + part[4 * jj + 3][rr]);
        if (jo < r && row0 + rr < m) store_t(t, static_cast<size_t>(row0 + rr) * r + jo, v * scale, bf16_out);
    }
}

__device__ __forceinline__ float lora_dot(const float *t, const __nv_bfloat16 *b, int r) {
    float d = 0.f;
    for (int j = 0; j < r; j += 2) {
        const uint32_t w = *reinterpret_cast<const uint32_t *>(b + j);
        d += t[j] * __uint_as_float(w << 16) + t[j + 1] * __uint_as_float(w & 0xFFFF0000u);
    }
    return d;
}

// One thread per output element of C ([m, n], or [m, n/2] with SwiGLU).
__global__ void __launch_bounds__(256) finish_kernel(const __nv_bfloat16 *__restrict__ base, __nv_bfloat16 *__restrict__ c, int m,
                                                     int n, const float *__restrict__ t, const __nv_bfloat16 *__restrict__ lb, int r,
                                                     int swiglu) {
    const int n_out = swiglu ? n / 2 : n;
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<size_t>(m) * n_out) return;
    const int row = static_cast<int>(idx / n_out), oc = static_cast<int>(idx - static_cast<size_t>(row) * n_out);
    auto value = [&](int col) {
        float v = __bfloat162float(base[static_cast<size_t>(row) * n + col]);
        if (r) v += lora_dot(t + static_cast<size_t>(row) * r, lb + static_cast<size_t>(col) * r, r);
        return v;
    };
    if (!swiglu) {
        c[idx] = __float2bfloat16(value(oc));
    } else {
        const int cg = (oc >> 5) * 64 + (oc & 31);  // gate column; its up column is 32 further
        const float g = value(cg), u = value(cg + 32);
        c[idx] = __float2bfloat16(g / (1.f + __expf(-g)) * u);
    }
}

}  // namespace

int launch_lora_down(const void *x, const void *lora_a, float scale, int m, int k, int r, void *t, int bf16_out, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    const bool rows8 = m > 32;
    cfg.gridDim = rows8 ? dim3((r + 1) / 2, (m + 7) / 8, 1) : dim3((r + 7) / 8, m, 1);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (cfg.gridDim.y > 65535) return KILN_W4A16_ERR_KERN_SHAPE;
    note_launch();
    if (rows8)
        return record_cuda_error(cudaLaunchKernelEx(&cfg, lora_down_rows8_kernel, static_cast<const __nv_bfloat16 *>(x),
                                                    static_cast<const __nv_bfloat16 *>(lora_a), scale, m, k, r, t, bf16_out));
    return record_cuda_error(cudaLaunchKernelEx(&cfg, lora_down_kernel, static_cast<const __nv_bfloat16 *>(x),
                                                static_cast<const __nv_bfloat16 *>(lora_a), scale, k, r, t, bf16_out));
}

int launch_finish(const void *base, void *c, int m, int n, const float *t, const void *lora_b, int r, int swiglu,
                  cudaStream_t stream) {
    const size_t total = static_cast<size_t>(m) * (swiglu ? n / 2 : n);
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    note_launch();
    finish_kernel<<<blocks, 256, 0, stream>>>(static_cast<const __nv_bfloat16 *>(base), static_cast<__nv_bfloat16 *>(c), m, n, t,
                                              static_cast<const __nv_bfloat16 *>(lora_b), r, swiglu);
    return record_cuda_error(cudaGetLastError());
}

}  // namespace kiln
