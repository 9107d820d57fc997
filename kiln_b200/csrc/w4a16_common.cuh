// Shared device helpers and host-side declarations for the W4A16 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/kiln_w4a16.h"

namespace kiln {

// ---- Marlin layout facts (what the packer of kiln-marlin-gemm/src/lib.rs:429-479 emits) ----
// b_packed is [k/16][n/64][32 lanes][4 words]: one 512-byte block per (16 K-rows, 64 N-cols).
// In a block, lane l (qd = l%4, c = l/4) owns four words, word j covering the 16-column tile
// j of the chunk.  Nibble i of a word holds q[kb*16 + r][chunk*64 + j*16 + cc] for
//   (r, cc) = (2qd, c) (2qd+8, c) (2qd, c+8) (2qd+8, c+8) (2qd+1, c) (2qd+9, c) (2qd+1, c+8) (2qd+9, c+8)
// so nibbles (0,4), (1,5), (2,6), (3,7) are the four bf16x2 B registers of two m16n8k16 MMAs.
// Grouped scales: within every 64 columns, position 8*i + j holds column i + 8*j.
constexpr int kGroup = 128;     // K elements per scale group
constexpr int kChunkCols = 64;  // N columns per 512-byte block

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(x), "r"(mask), "r"(orv));
    return r;
}

// bf16 has 7 mantissa bits: OR-ing a nibble into the low mantissa bits of 128.0 (0x4300)
// gives exactly 128 + v.
constexpr uint32_t kNibMask = 0x000F000Fu;
constexpr uint32_t kMagic128 = 0x43004300u;  // bf16x2 {128, 128}
constexpr uint32_t kNeg136x2 = 0xC308C308u;  // bf16x2 {-136, -136} = -(128 + 8)
constexpr uint32_t kPos136x2 = 0x43084308u;  // bf16x2 {136, 136}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_addr));
}

// Weights are read exactly once: bypass L1.
__device__ __forceinline__ uint4 ld_stream_v4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Activations: cached in L2 only, so a buffer another kernel has just rewritten is never read from a stale L1 line.
__device__ __forceinline__ uint4 ld_cg_v4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Programmatic dependent launch: let the next kernel in the stream start its prologue,
// and wait for the previous kernel's memory before touching anything it may have written.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta));
    return r;
}
__device__ __forceinline__ float2 ld_dsmem_f2(uint32_t cluster_addr) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(cluster_addr));
    return v;
}

__device__ __forceinline__ void st_dsmem_f2(uint32_t cluster_addr, float2 v) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1,%2};" ::"r"(cluster_addr), "f"(v.x), "f"(v.y) : "memory");
}

// Position of natural column `col` inside the per-column (groupsize -1) scale order
// (kiln-marlin-gemm/src/lib.rs:348-357): within each 32, out[8i + j] = in[2i + {0,1,8,9,16,17,24,25}[j]].
__device__ __host__ __forceinline__ int scale_single_pos(int col) {
    int c32 = col & 31;
    return (col & ~31) + 8 * ((c32 & 7) >> 1) + 2 * (c32 >> 3) + (c32 & 1);
}

// ---- host side --------------------------------------------------------------------------
struct GemmArgs {
    const void *A;   // bf16 [m,k]
    const void *B;   // int32 [k/16, 2n]
    const void *S;   // fp16 [k/g, n]
    void *C;         // bf16 [m,n]
    int m, n, k;
    int groupsize;   // 128 or -1
    void *workspace;
    size_t workspace_bytes;
    cudaStream_t stream;
    // fused all-gather (prefill kernel only): store the result into the row-major [m, ldc] buffers of n_peers GPUs
    void *peer_c[8] = {};
    int n_peers = 0, ldc = 0, col0 = 0;
    // the same with one NVSwitch multicast address for the whole group instead of per-GPU pointers (multimem.st)
    void *mc_c = nullptr;
    // epilogue options (LoRA: decode kernel; SwiGLU: decode kernel, and the tcgen05 kernel's whole-tile tilings): LoRA delta C += lora_t * lora_b^T with lora_t [m, lora_r] = scale * x * A^T (fp32 for the decode kernel, bf16 for the tcgen05 kernel)
    // and lora_b bf16 [n, lora_r]; swiglu: columns are gate/up interleaved in runs of 32, C is [m, n/2]
    bool no_scratch = false;  // the tcgen05 kernel may not use the workspace (legacy entry point: its caller's buffer is tiny)
    const void *lora_t = nullptr;
    const void *lora_b = nullptr;
    int lora_r = 0;
    int swiglu = 0;
};

// One GEMM of a grouped decode launch.
struct DecodeItem {
    const void *A, *B, *S;
    void *C;
    int m, n, k, groupsize;
    const void *lora_t, *lora_b;
    int lora_r, swiglu;
};

struct DecodeOverride {
    int cluster_k, warps_k, warps_n;
};

int device_sm_count();
void note_launch(unsigned n = 1);
int record_cuda_error(cudaError_t e);  // returns KILN_W4A16_ERR_CUDA if e != success else 0
uint32_t *device_status_word();        // per-device word written by bounded waits; nullptr on failure

int launch_decode(const GemmArgs &a, const DecodeOverride &ov);
void decode_plan(int m, int n, int k, const DecodeOverride &ov, int out[4]);
int launch_decode_list(const DecodeItem *items, int count, cudaStream_t stream, const DecodeOverride &ov);
int launch_lora_down(const void *x, const void *lora_a, float scale, int m, int k, int r, void *t, int bf16_out, cudaStream_t stream);
bool prefill_fuses_lora(int groupsize, int lora_r);
int launch_finish(const void *base, void *c, int m, int n, const float *t, const void *lora_b, int r, int swiglu, cudaStream_t stream);
int launch_prefill(const GemmArgs &a);
size_t prefill_workspace_bytes(int m, int n, int k);
void set_prefill_override(int bn, int splits, int mt, int stream_k);
void set_wait_limit_ns(unsigned long long ns);
unsigned long long current_wait_limit_ns();
void set_smallm_enabled(int on);
bool smallm_supported(int m, int n, int k, int groupsize);
int launch_smallm(const GemmArgs &a, int splits, float *partial);
void set_test_drop_a_load(int k_step);
void prefill_plan(int m, int n, int k, int out[4]);
bool prefill_supported(int m, int n, int k, int groupsize);
bool prefill_fuses_swiglu(int m, int n, int k);
int static_status_read_clear(cudaStream_t st, uint32_t *out);
int decode_status_read_clear(cudaStream_t st, uint32_t *out);

}  // namespace kiln
