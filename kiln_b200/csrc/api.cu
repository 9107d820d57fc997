// C ABI, argument validation and kernel selection for the W4A16 GEMM.
//
// Mirrors, under the C boundary, what the reference does in its Rust wrapper
// (kiln-marlin-gemm/src/lib.rs:97-275: shape and groupsize checks, workspace sizing,
// status mapping) and in its host dispatcher (kiln-marlin-gemm/csrc/marlin_kernel.cu:731-819:
// shape -> kernel/tile choice), so that both are testable without a Rust toolchain.
#include <atomic>
#include <mutex>

#include "w4a16_common.cuh"

namespace kiln {

namespace {
std::atomic<unsigned long long> g_launches{0};
thread_local int t_last_cuda_error = 0;
DecodeOverride g_decode_override{0, 0, 0};
constexpr int kDefaultPrefillMinM = 0;  // 0 = the built-in rule
std::atomic<int> g_prefill_min_m{kDefaultPrefillMinM};
}  // namespace

void note_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int record_cuda_error(cudaError_t e) {
    if (e == cudaSuccess) return 0;
    t_last_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();  // clear the sticky-less error so the next call starts clean
    return KILN_W4A16_ERR_CUDA;
}

int device_sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int sms = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
        cached[dev] = sms;
    }
    return cached[dev];
}

// One status word per device, in its own small allocation made on first use (outside any
// stream capture: call the GEMM once before capturing).
uint32_t *device_status_word() {
    static uint32_t *words[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        uint32_t *p = nullptr;
        if (record_cuda_error(cudaMalloc(&p, 256))) return nullptr;
        if (record_cuda_error(cudaMemset(p, 0, 256))) return nullptr;
        words[dev] = p;
    }
    return words[dev];
}

static int validate(const GemmArgs &a) {
    if (a.m < 0 || a.n < 0 || a.k < 0) return KILN_W4A16_ERR_ARG;
    // kiln-marlin-gemm/src/lib.rs:112-117, 128-142
    if (a.k % 128 != 0 || a.n % 256 != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    if (!(a.groupsize == -1 || a.groupsize == 128)) return KILN_W4A16_ERR_PROB_SHAPE;
    if (a.m == 0 || a.n == 0 || a.k == 0) return KILN_W4A16_OK;  // marlin_kernel.cu:772-773
    if (!a.A || !a.B || !a.C || !a.S) return KILN_W4A16_ERR_ARG;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B) |
                           reinterpret_cast<uintptr_t>(a.C) | reinterpret_cast<uintptr_t>(a.S) |
                           reinterpret_cast<uintptr_t>(a.workspace);
    if (bits & 15) return KILN_W4A16_ERR_ALIGNMENT;
    return -1;  // proceed
}

// Kernel choice (measured on B200, CUDA-graph replay over rotating weights).  The decode kernel handles 8 or 16 rows per
// block of CTAs and repeats the int4 dequant for every block; the tcgen05 kernel dequantises once per 128 rows but pays
// a fixed cost per launch and per K-step of a tile.  Measured crossovers (decode / tcgen05, us):
//  * wide projections (4096 columns and more): the decode kernel wins up to 32 rows, two blocks of 16 (gate+up M=32:
//    19.2 / 16.4 but M=24: 18.8 / 22.7; q M=32: 8.2 / 8.9; GDN-in M=32: 11.8 / 11.6), a third block costs it far more than
//    a tile (gate+up M=40: 32.3 / 16.4, q: 12.7 / 9.4);
//  * projections of about 2560 columns have few column blocks for the decode kernel to spread over: the tcgen05 kernel
//    wins from 17 rows (down M=17: 13.4 / 11.8, M=32: 13.7 / 12.5; o M=17: 9.5 / 8.2, M=32: 9.9 / 8.9, M=64: 14.4 / 11.2),
//    provided the activation matrix is at least 128 KB (smaller ones were measured 40 % slower through its TMA loads);
//  * projections of 1024 columns or fewer (k, v: four to eight tiles) stay on the decode kernel up to M = 256
//    (k at M=128: 6.4 / 15.3).
//  * a GEMM without epilogue options and at most 128 rows runs on the tcgen05 kernel that keeps the
//    weights in tensor memory (smallm_w4a16_tmem.cu), which moves the crossover to 17 rows for every projection of more
//    than 1024 columns (M=17: q 7.8 / 6.8, gate+up 18.3 / 13.6, down 12.8 / 10.1, GDN-in 11.0 / 10.0, o 9.1 / 7.0;
//    M=16, one block of the decode kernel: q 5.7 / 6.6, gate+up 12.0 / 13.4).
// kiln_w4a16_set_prefill_min_m replaces the rule by a plain threshold.
static bool use_prefill(int m, int n, int k, int groupsize, bool plain = false) {
    if (!prefill_supported(m, n, k, groupsize)) return false;
    const int min_m = g_prefill_min_m.load(std::memory_order_relaxed);
    if (min_m != kDefaultPrefillMinM) return m >= min_m;
    if (n <= 1024) return m > 256;
    if (plain && m <= 64 && smallm_supported(m, n, k, groupsize)) return m >= 17;
    if (n <= 3072 && static_cast<long long>(m) * k * 2 >= (128LL << 10)) return m >= 17;
    return m >= 33;
}

// no epilogue option and no fused all-gather: what the small-batch tcgen05 kernel takes
static bool plain_gemm(const GemmArgs &a) { return !a.swiglu && a.lora_r == 0 && a.n_peers == 0 && !a.mc_c && !a.no_scratch; }

static int gemm(const GemmArgs &a) {
    const int v = validate(a);
    if (v >= 0) return v;
    if (use_prefill(a.m, a.n, a.k, a.groupsize, plain_gemm(a))) {
        const size_t need = a.no_scratch ? 0 : prefill_workspace_bytes(a.m, a.n, a.k);
        if (need > 0 && (!a.workspace || a.workspace_bytes < need)) return KILN_W4A16_ERR_WORKSPACE;
        return launch_prefill(a);
    }
    return launch_decode(a, g_decode_override);
}

}  // namespace kiln

using namespace kiln;

extern "C" {

kiln_w4a16_status_t kiln_w4a16_gemm_bf16(const void *A, const void *B, void *C, const void *s, int m, int n,
                                         int k, int groupsize, void *workspace, size_t workspace_bytes,
                                         void *stream) {
    GemmArgs a{A, B, s, C, m, n, k, groupsize, workspace, workspace_bytes, static_cast<cudaStream_t>(stream)};
    return gemm(a);
}

kiln_w4a16_status_t kiln_marlin_w4a16_gemm(const void *A, const void *B, void *C, void *s, int prob_m,
                                           int prob_n, int prob_k, void *workspace, int groupsize, int dev,
                                           void *stream, int thread_k, int thread_n, int sms, int max_par) {
    (void)dev;
    (void)sms;
    (void)max_par;
    // The reference rejects tile overrides the problem is not a multiple of
    // (marlin_kernel.cu:770-771) and tuples it has no kernel for (:811-812).
    if (thread_k != -1 || thread_n != -1) {
        const bool known = (thread_k == 128 && thread_n == 128) || (thread_k == 64 && thread_n == 256);
        if (thread_k <= 0 || thread_n <= 0) return KILN_W4A16_ERR_KERN_SHAPE;
        if (prob_n % thread_n != 0 || prob_k % thread_k != 0) return KILN_W4A16_ERR_PROB_SHAPE;
        if (!known) return KILN_W4A16_ERR_KERN_SHAPE;
    }
    // The legacy signature carries no size, and an unmodified reference wrapper passes its lock array of
    // (n / 128) * 16 int32 (kiln-marlin-gemm/src/lib.rs:174-178): this entry therefore never writes to `workspace`.  The
    // tcgen05 kernel is restricted to tilings without split-K or stream-K here; the faster tilings need
    // kiln_w4a16_gemm_bf16, whose workspace size is checked.
    (void)workspace;
    GemmArgs a{A, B, s, C, prob_m, prob_n, prob_k, groupsize, nullptr, 0, static_cast<cudaStream_t>(stream)};
    a.no_scratch = true;
    return gemm(a);
}

kiln_w4a16_status_t kiln_w4a16_gemm_bf16_allgather(const void *A, const void *B, const void *s, int m, int n_local,
                                                   int k, int groupsize, void *const *C_peers, int n_peers, int ldc,
                                                   int col0, void *stream) {
    if (!C_peers || n_peers < 1 || n_peers > 8) return KILN_W4A16_ERR_ARG;
    if (ldc < col0 + n_local || col0 < 0 || ldc % 8 != 0 || col0 % 8 != 0) return KILN_W4A16_ERR_ARG;
    GemmArgs a{A, B, s, C_peers[0], m, n_local, k, groupsize, nullptr, 0, static_cast<cudaStream_t>(stream)};
    const int v = validate(a);
    if (v >= 0) return v;
    if (!prefill_supported(m, n_local, k, groupsize)) return KILN_W4A16_ERR_KERN_SHAPE;
    for (int i = 0; i < n_peers; ++i) {
        if (!C_peers[i]) return KILN_W4A16_ERR_ARG;
        if (reinterpret_cast<uintptr_t>(C_peers[i]) & 15) return KILN_W4A16_ERR_ALIGNMENT;
        a.peer_c[i] = C_peers[i];
    }
    a.n_peers = n_peers;
    a.ldc = ldc;
    a.col0 = col0;
    return launch_prefill(a);
}

kiln_w4a16_status_t kiln_w4a16_gemm_bf16_allgather_multicast(const void *A, const void *B, const void *s, int m,
                                                             int n_local, int k, int groupsize, void *C_multicast,
                                                             int ldc, int col0, void *stream) {
    if (ldc < col0 + n_local || col0 < 0 || ldc % 8 != 0 || col0 % 8 != 0) return KILN_W4A16_ERR_ARG;
    GemmArgs a{A, B, s, C_multicast, m, n_local, k, groupsize, nullptr, 0, static_cast<cudaStream_t>(stream)};
    const int v = validate(a);
    if (v >= 0) return v;
    if (!prefill_supported(m, n_local, k, groupsize)) return KILN_W4A16_ERR_KERN_SHAPE;
    a.mc_c = C_multicast;
    a.ldc = ldc;
    a.col0 = col0;
    return launch_prefill(a);
}

namespace {
size_t align256(size_t x) { return (x + 255) / 256 * 256; }

int validate_epilogue(const kiln_w4a16_epilogue_t *ep, int n) {
    if (!ep) return KILN_W4A16_OK;
    if (ep->swiglu && n % 128 != 0) return KILN_W4A16_ERR_PROB_SHAPE;
    if (ep->lora_rank < 0 || ep->lora_rank > 128 || ep->lora_rank % 8 != 0) return KILN_W4A16_ERR_ARG;
    if (ep->lora_rank && (!ep->lora_a || !ep->lora_b)) return KILN_W4A16_ERR_ARG;
    if (ep->lora_rank && ((reinterpret_cast<uintptr_t>(ep->lora_a) | reinterpret_cast<uintptr_t>(ep->lora_b)) & 15))
        return KILN_W4A16_ERR_ALIGNMENT;
    return KILN_W4A16_OK;
}
}  // namespace

// SwiGLU alone, fused by the tcgen05 kernel that would run it: the kernel choice is the plain GEMM's (from 17 rows)
static bool ex_plain(const kiln_w4a16_epilogue_t *ep, int m, int n, int k) {
    return ep->lora_rank == 0 && ep->swiglu && m <= 128 && prefill_fuses_swiglu(m, n, k);
}

size_t kiln_w4a16_workspace_bytes_ex(int m, int n, int k, const kiln_w4a16_epilogue_t *ep) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    const bool opts = ep && (ep->swiglu || ep->lora_rank);
    if (!opts) return kiln_w4a16_workspace_bytes(m, n, k);
    size_t need = align256(static_cast<size_t>(m) * ep->lora_rank * sizeof(float));
    if (use_prefill(m, n, k, 128, ex_plain(ep, m, n, k))) {
        // tcgen05 kernel: SwiGLU is fused when the tiling writes whole tiles, the LoRA delta whenever the scales are grouped
        // (this call does not know the group size, so it reserves the composed path's buffer whenever there is a delta);
        // what is not fused is applied by a second pass over the bf16 GEMM result kept in the workspace
        const bool composed = (ep->swiglu && !prefill_fuses_swiglu(m, n, k)) || ep->lora_rank;
        if (composed) need += align256(static_cast<size_t>(m) * n * 2);
        need += align256(prefill_workspace_bytes(m, n, k));
    }
    return need;
}

kiln_w4a16_status_t kiln_w4a16_gemm_bf16_ex(const void *A, const void *B, void *C, const void *s, int m, int n, int k,
                                            int groupsize, const kiln_w4a16_epilogue_t *ep, void *workspace,
                                            size_t workspace_bytes, void *stream) {
    const bool opts = ep && (ep->swiglu || ep->lora_rank);
    if (!opts) return kiln_w4a16_gemm_bf16(A, B, C, s, m, n, k, groupsize, workspace, workspace_bytes, stream);
    if (int rc = validate_epilogue(ep, n)) return rc;
    GemmArgs a{A, B, s, C, m, n, k, groupsize, workspace, workspace_bytes, static_cast<cudaStream_t>(stream)};
    const int v = validate(a);
    if (v >= 0) return v;
    const size_t need = kiln_w4a16_workspace_bytes_ex(m, n, k, ep);
    if (need > 0 && (!workspace || workspace_bytes < need)) return KILN_W4A16_ERR_WORKSPACE;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    const bool tc = use_prefill(m, n, k, groupsize, ex_plain(ep, m, n, k));
    const bool fuse_lora = tc && ep->lora_rank && prefill_fuses_lora(groupsize, ep->lora_rank);
    const bool fuse_swiglu = tc && ep->swiglu && prefill_fuses_swiglu(m, n, k);
    void *t = nullptr;
    if (ep->lora_rank) {
        t = ws;  // fp32 [m, r] for the decode kernel and the composed pass, bf16 [m, r] as an operand of the tcgen05 kernel
        ws += align256(static_cast<size_t>(m) * ep->lora_rank * sizeof(float));
        if (int rc = launch_lora_down(A, ep->lora_a, ep->lora_scale, m, k, ep->lora_rank, t, fuse_lora ? 1 : 0, a.stream)) return rc;
    }
    if (!tc) {
        a.lora_t = t;
        a.lora_b = ep->lora_b;
        a.lora_r = ep->lora_rank;
        a.swiglu = ep->swiglu ? 1 : 0;
        return launch_decode(a, g_decode_override);
    }
    const bool composed = (ep->swiglu && !fuse_swiglu) || (ep->lora_rank && !fuse_lora);
    void *tmp = nullptr;
    if (composed) {
        tmp = ws;
        ws += align256(static_cast<size_t>(m) * n * 2);
    }
    GemmArgs b{A, B, s, composed ? tmp : C, m, n, k, groupsize, ws, prefill_workspace_bytes(m, n, k), a.stream};
    if (fuse_lora) {
        b.lora_t = t;
        b.lora_b = ep->lora_b;
        b.lora_r = ep->lora_rank;
    }
    if (!composed && fuse_swiglu) b.swiglu = 1;
    if (int rc = launch_prefill(b)) return rc;
    if (!composed) return KILN_W4A16_OK;
    return launch_finish(tmp, C, m, n, fuse_lora ? nullptr : static_cast<const float *>(t), ep->lora_b, fuse_lora ? 0 : ep->lora_rank,
                         ep->swiglu ? 1 : 0, a.stream);
}

kiln_w4a16_status_t kiln_w4a16_gemm_bf16_grouped(const kiln_w4a16_problem_t *problems, int count, void *workspace,
                                                 size_t workspace_bytes, void *stream) {
    if (!problems || count < 1 || count > KILN_W4A16_MAX_GROUP) return KILN_W4A16_ERR_ARG;
    DecodeItem items[KILN_W4A16_MAX_GROUP] = {};
    bool one_launch = true;
    int live = 0;
    for (int i = 0; i < count; ++i) {
        const kiln_w4a16_problem_t &q = problems[i];
        GemmArgs a{q.A, q.B, q.s, q.C, q.m, q.n, q.k, q.groupsize, workspace, workspace_bytes, static_cast<cudaStream_t>(stream)};
        const int v = validate(a);
        if (v > 0) return v;
        if (v == 0) continue;  // an empty problem
        if (use_prefill(q.m, q.n, q.k, q.groupsize)) one_launch = false;  // (one decode launch for the group beats per-problem small-batch launches)
        items[live++] = DecodeItem{q.A, q.B, q.s, q.C, q.m, q.n, q.k, q.groupsize, nullptr, nullptr, 0, 0};
    }
    if (live == 0) return KILN_W4A16_OK;
    // one batch class per launch: up to 8 rows, or 9 and more
    for (int i = 1; i < live; ++i)
        if ((items[i].m <= 8) != (items[0].m <= 8)) one_launch = false;
    if (one_launch) return launch_decode_list(items, live, static_cast<cudaStream_t>(stream), g_decode_override);
    for (int i = 0; i < live; ++i) {  // batch sizes of the tcgen05 kernel, or mixed classes: one launch each
        const DecodeItem &q = items[i];
        if (int rc = kiln_w4a16_gemm_bf16(q.A, q.B, q.C, q.S, q.m, q.n, q.k, q.groupsize, workspace, workspace_bytes, stream))
            return rc;
    }
    return KILN_W4A16_OK;
}

size_t kiln_w4a16_workspace_bytes(int m, int n, int k) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    if (use_prefill(m, n, k, 128, true)) return prefill_workspace_bytes(m, n, k);
    return 0;
}

int kiln_w4a16_shape_is_supported(int k, int n) { return k > 0 && n > 0 && k % 128 == 0 && n % 256 == 0; }

int kiln_w4a16_last_cuda_error(void) { return t_last_cuda_error; }

kiln_w4a16_status_t kiln_w4a16_check_device_status(void *stream, uint32_t *detail) {
    uint32_t *w = device_status_word();
    if (!w) return KILN_W4A16_ERR_CUDA;
    uint32_t host = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int rc = record_cuda_error(cudaMemcpyAsync(&host, w, sizeof(host), cudaMemcpyDeviceToHost, st))) return rc;
    if (int rc = record_cuda_error(cudaStreamSynchronize(st))) return rc;
    uint32_t host_static = 0;  // the word of the no-allocation entry's launches (kept in the library image)
    if (int rc = static_status_read_clear(st, &host_static)) return rc;
    uint32_t host_decode = 0;  // the decode kernel's word (split-K exchange between the CTAs of a cluster)
    if (int rc = decode_status_read_clear(st, &host_decode)) return rc;
    if (detail) *detail = host ? host : (host_static ? host_static : host_decode);
    if (host != 0) {
        if (int rc = record_cuda_error(cudaMemsetAsync(w, 0, sizeof(uint32_t), st))) return rc;
        if (int rc = record_cuda_error(cudaStreamSynchronize(st))) return rc;
    }
    return (host | host_static | host_decode) ? KILN_W4A16_ERR_TIMEOUT : KILN_W4A16_OK;
}

void kiln_w4a16_set_decode_override(int cluster_k, int warps_k, int warps_n) {
    g_decode_override = DecodeOverride{cluster_k, warps_k, warps_n};
}

void kiln_w4a16_decode_plan(int m, int n, int k, int out[4]) {
    if (out && m > 0 && n > 0 && k > 0) decode_plan(m, n, k, g_decode_override, out);
}

void kiln_w4a16_set_small_batch_kernel(int enabled) { set_smallm_enabled(enabled); }

void kiln_w4a16_set_prefill_override(int bn, int splits, int m_tiles, int stream_k) {
    set_prefill_override(bn, splits, m_tiles, stream_k);
}

void kiln_w4a16_set_wait_limit_ns(unsigned long long ns) { set_wait_limit_ns(ns); }

void kiln_w4a16_test_drop_activation_load(int k_step) { set_test_drop_a_load(k_step); }

void kiln_w4a16_prefill_plan(int m, int n, int k, int out[4]) {
    if (out) prefill_plan(m, n, k, out);
}

void kiln_w4a16_set_prefill_min_m(int min_m) {
    g_prefill_min_m.store(min_m > 0 ? min_m : kDefaultPrefillMinM, std::memory_order_relaxed);
}

int kiln_w4a16_version(void) { return 100; }

unsigned long long kiln_w4a16_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
