//! W4A16 GEMM for B200 behind the public API of kiln's `kiln-marlin-gemm` crate.
//!
//! Same two entry points as the crate it replaces: [`marlin_w4a16_gemm`] and [`pack`].
//! Everything that computes lives under the C ABI of `include/kiln_w4a16.h`; this file only
//! validates shapes the way the original wrapper does, borrows device pointers from candle
//! and forwards them.  Differences from the original wrapper are all removals: no bf16<->fp16
//! casts (the kernels read and write bf16), no zeroed lock buffer per call (split-K scratch is
//! a per-device buffer that is created once, grows when a larger problem needs it and is never
//! cleared; batch sizes below 33 need none), no hard-coded device 0.  The output tensor is still
//! created with `Tensor::zeros`, as in the original: candle offers no safe uninitialised
//! constructor, and the kernels overwrite every element.
//!
//! NOTE: authored without a Rust toolchain at hand; it has not been compiled.

use candle_core::{
    backend::BackendStorage, cuda_backend::cudarc::driver::DevicePtr, DType, Result, Tensor,
};
use half::f16;
use std::ffi::c_void;
use std::sync::Mutex;

/// Split-K scratch, one buffer per CUDA device ordinal, kept for the life of the process.  The kernels
/// neither expect it to be zero nor leave anything in it that a later call reads.  Calls on one device
/// are expected on one stream (candle's), as in the original wrapper.
static WORKSPACES: Mutex<Vec<(usize, Tensor)>> = Mutex::new(Vec::new());

fn workspace_for(device: &candle_core::Device, ordinal: usize, bytes: usize) -> Result<Tensor> {
    let mut all = WORKSPACES.lock().unwrap();
    if let Some((_, t)) = all.iter().find(|(o, t)| *o == ordinal && t.elem_count() >= bytes) {
        return Ok(t.clone());
    }
    let t = Tensor::zeros((bytes.max(1 << 20),), DType::U8, device)?;
    all.retain(|(o, _)| *o != ordinal);
    all.push((ordinal, t.clone()));
    Ok(t)
}

unsafe extern "C" {
    fn kiln_w4a16_gemm_bf16(
        a: *const c_void,
        b: *const c_void,
        c: *mut c_void,
        s: *const c_void,
        m: i32,
        n: i32,
        k: i32,
        groupsize: i32,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: *mut c_void,
    ) -> i32;
    fn kiln_w4a16_workspace_bytes(m: i32, n: i32, k: i32) -> usize;
    fn kiln_w4a16_quantize_and_pack_host(
        weight: *const f32,
        k: i32,
        n: i32,
        groupsize: i32,
        b_packed: *mut i32,
        scales_f16: *mut u16,
        dequant: *mut f32,
        num_threads: i32,
    ) -> i32;
    fn kiln_w4a16_build_weight_perm(out: *mut i32);
    fn kiln_w4a16_build_scale_perm(out: *mut i32);
    fn kiln_w4a16_build_scale_perm_single(out: *mut i32);
    // Beyond the original crate (declared for callers that want them; see include/kiln_w4a16.h):
    /// quantise + pack on the device, straight from the bf16 / f32 `[k, n]` weight in HBM
    pub fn kiln_w4a16_quantize_and_pack_device(
        weight: *const c_void,
        weight_is_bf16: i32,
        k: i32,
        n: i32,
        groupsize: i32,
        b_packed: *mut i32,
        scales_f16: *mut u16,
        dequant: *mut f32,
        stream: *mut c_void,
    ) -> i32;
    /// GPTQ `qweight` / `qzeros` / `scales` -> this format without dequantising (symmetric checkpoints only)
    pub fn kiln_w4a16_repack_gptq_device(
        qweight: *const i32,
        qzeros: *const i32,
        scales: *const u16,
        k: i32,
        n: i32,
        groupsize: i32,
        b_packed: *mut i32,
        scales_perm: *mut u16,
        asymmetric: *mut u32,
        stream: *mut c_void,
    ) -> i32;
    /// the GEMM with epilogue options: LoRA delta and / or SwiGLU of an interleaved gate+up matrix
    pub fn kiln_w4a16_gemm_bf16_ex(
        a: *const c_void,
        b: *const c_void,
        c: *mut c_void,
        s: *const c_void,
        m: i32,
        n: i32,
        k: i32,
        groupsize: i32,
        epilogue: *const KilnW4a16Epilogue,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: *mut c_void,
    ) -> i32;
    pub fn kiln_w4a16_workspace_bytes_ex(m: i32, n: i32, k: i32, epilogue: *const KilnW4a16Epilogue) -> usize;
    /// several independent GEMMs (q, k, v of a layer) in one launch at decode batch sizes
    pub fn kiln_w4a16_gemm_bf16_grouped(
        problems: *const KilnW4a16Problem,
        count: i32,
        workspace: *mut c_void,
        workspace_bytes: usize,
        stream: *mut c_void,
    ) -> i32;
    /// column-parallel GEMM whose epilogue stores into every GPU's `[m, ldc]` buffer
    pub fn kiln_w4a16_gemm_bf16_allgather(
        a: *const c_void,
        b: *const c_void,
        s: *const c_void,
        m: i32,
        n_local: i32,
        k: i32,
        groupsize: i32,
        c_peers: *const *mut c_void,
        n_peers: i32,
        ldc: i32,
        col0: i32,
        stream: *mut c_void,
    ) -> i32;
}

/// `kiln_w4a16_epilogue_t` of include/kiln_w4a16.h.
#[repr(C)]
pub struct KilnW4a16Epilogue {
    pub swiglu: i32,
    pub lora_a: *const c_void,
    pub lora_b: *const c_void,
    pub lora_rank: i32,
    pub lora_scale: f32,
}

/// `kiln_w4a16_problem_t` of include/kiln_w4a16.h.
#[repr(C)]
pub struct KilnW4a16Problem {
    pub a: *const c_void,
    pub b: *const c_void,
    pub c: *mut c_void,
    pub s: *const c_void,
    pub m: i32,
    pub n: i32,
    pub k: i32,
    pub groupsize: i32,
}

/// `a [m,k] bf16` x `b_packed [k/16, n*16/8] i32` x `scales [k/groupsize, n] f16` -> `[m,n] bf16`.
/// Constraints and error messages follow the original wrapper.
pub fn marlin_w4a16_gemm(
    a: &Tensor,
    b_packed: &Tensor,
    scales: &Tensor,
    groupsize: i32,
) -> Result<Tensor> {
    let device = a.device();
    if !device.is_cuda() {
        candle_core::bail!("kiln-marlin-gemm: a must be on CUDA");
    }
    let (m, k) = a.dims2()?;
    let (b_rows, b_cols) = b_packed.dims2()?;
    let (s_rows, n) = scales.dims2()?;
    if k % 128 != 0 {
        candle_core::bail!("kiln-marlin-gemm: k must be a multiple of 128 (got {k})");
    }
    if n % 256 != 0 {
        candle_core::bail!("kiln-marlin-gemm: n must be a multiple of 256 (got {n})");
    }
    if b_rows != k / 16 || b_cols != n * 16 / 8 {
        candle_core::bail!(
            "kiln-marlin-gemm: b_packed shape [{b_rows}, {b_cols}] does not match expected \
             [k/16={}, n*16/8={}] for k={k}, n={n}",
            k / 16,
            n * 16 / 8,
        );
    }
    if !(groupsize == -1 || groupsize == 128) {
        candle_core::bail!("kiln-marlin-gemm: groupsize must be -1 or 128 (got {groupsize})");
    }
    let g: usize = if groupsize == -1 { k } else { groupsize as usize };
    if g > k || k % g != 0 {
        candle_core::bail!("kiln-marlin-gemm: k={k} must be divisible by groupsize={groupsize}");
    }
    if s_rows != k / g {
        candle_core::bail!(
            "kiln-marlin-gemm: scales rows {s_rows} != expected {} (k={k}, groupsize={groupsize})",
            k / g
        );
    }
    if a.dtype() != DType::BF16 {
        candle_core::bail!("kiln-marlin-gemm: a must be bf16 (got {:?})", a.dtype());
    }
    if b_packed.dtype() != DType::I32 {
        candle_core::bail!("kiln-marlin-gemm: b_packed must be i32 (got {:?})", b_packed.dtype());
    }
    if scales.dtype() != DType::F16 {
        candle_core::bail!("kiln-marlin-gemm: scales must be f16 (got {:?})", scales.dtype());
    }

    let a = a.contiguous()?;
    let b_packed = b_packed.contiguous()?;
    let scales = scales.contiguous()?;
    // fully overwritten by the kernel; zeros() only because candle has no uninitialised constructor here
    let c = Tensor::zeros((m, n), DType::BF16, device)?;
    let ws_bytes = unsafe { kiln_w4a16_workspace_bytes(m as i32, n as i32, k as i32) };
    let ordinal = match device {
        candle_core::Device::Cuda(d) => d.ordinal(),
        _ => 0,
    };
    let ws = workspace_for(device, ordinal, ws_bytes.max(16))?;

    {
        let (a_st, a_l) = a.storage_and_layout();
        let (b_st, b_l) = b_packed.storage_and_layout();
        let (c_st, c_l) = c.storage_and_layout();
        let (s_st, s_l) = scales.storage_and_layout();
        let (w_st, w_l) = ws.storage_and_layout();
        macro_rules! cuda {
            ($st:expr, $what:literal) => {
                match &*$st {
                    candle_core::Storage::Cuda(c) => c,
                    _ => candle_core::bail!(concat!("kiln-marlin-gemm: ", $what, " must be on CUDA")),
                }
            };
        }
        let (a_c, b_c, c_c, s_c, w_c) = (
            cuda!(a_st, "a"),
            cuda!(b_st, "b_packed"),
            cuda!(c_st, "c"),
            cuda!(s_st, "scales"),
            cuda!(w_st, "workspace"),
        );
        let stream = a_c.device().cuda_stream();
        let raw_stream = stream.cu_stream() as *mut c_void;
        let a_s = a_c.as_cuda_slice::<half::bf16>()?.slice(a_l.start_offset()..);
        let b_s = b_c.as_cuda_slice::<i32>()?.slice(b_l.start_offset()..);
        let c_s = c_c.as_cuda_slice::<half::bf16>()?.slice(c_l.start_offset()..);
        let s_s = s_c.as_cuda_slice::<f16>()?.slice(s_l.start_offset()..);
        let w_s = w_c.as_cuda_slice::<u8>()?.slice(w_l.start_offset()..);
        unsafe {
            let (a_p, _g1) = a_s.device_ptr(&stream);
            let (b_p, _g2) = b_s.device_ptr(&stream);
            let (c_p, _g3) = c_s.device_ptr(&stream);
            let (s_p, _g4) = s_s.device_ptr(&stream);
            let (w_p, _g5) = w_s.device_ptr(&stream);
            let status = kiln_w4a16_gemm_bf16(
                a_p as *const _,
                b_p as *const _,
                c_p as *mut _,
                s_p as *const _,
                m as i32,
                n as i32,
                k as i32,
                groupsize,
                w_p as *mut _,
                ws_bytes,
                raw_stream,
            );
            if status != 0 {
                candle_core::bail!(
                    "kiln_marlin_w4a16_gemm failed with status {status} \
                     (1=ERR_PROB_SHAPE, 2=ERR_KERN_SHAPE) for m={m}, n={n}, k={k}, \
                     groupsize={groupsize}"
                );
            }
        }
    }
    Ok(c)
}

/// Same surface as the original `pack` module; the work is done by the native packer.
pub mod pack {
    use super::*;

    pub const MAX_Q: i32 = 15;
    pub const Q_OFFSET: i32 = 8;

    fn table(len: usize, f: unsafe extern "C" fn(*mut i32)) -> Vec<usize> {
        let mut raw = vec![0i32; len];
        unsafe { f(raw.as_mut_ptr()) };
        raw.into_iter().map(|v| v as usize).collect()
    }

    pub fn build_weight_perm() -> Vec<usize> {
        table(1024, kiln_w4a16_build_weight_perm)
    }

    pub fn build_scale_perm() -> Vec<usize> {
        table(64, kiln_w4a16_build_scale_perm)
    }

    pub fn build_scale_perm_single() -> Vec<usize> {
        table(32, kiln_w4a16_build_scale_perm_single)
    }

    /// `weight` row-major `[k, n]`; returns `(b_packed, scales, dequant)` exactly like the original.
    /// Single-threaded per call (`num_threads = 1`): kiln already fans projections out over rayon.
    pub fn quantize_and_pack(
        weight: &[f32],
        k: usize,
        n: usize,
        groupsize: i64,
    ) -> (Vec<i32>, Vec<f16>, Vec<f32>) {
        assert_eq!(weight.len(), k * n);
        assert_eq!(k % 128, 0, "k must be %128 == 0");
        assert_eq!(n % 256, 0, "n must be %256 == 0");
        let g = if groupsize == -1 { k } else { groupsize as usize };
        assert!(k % g == 0, "k={k} must be divisible by groupsize={g}");
        let mut packed = vec![0i32; (k / 16) * (2 * n)];
        let mut scales = vec![0u16; (k / g) * n];
        let mut dequant = vec![0f32; k * n];
        let rc = unsafe {
            kiln_w4a16_quantize_and_pack_host(
                weight.as_ptr(),
                k as i32,
                n as i32,
                groupsize as i32,
                packed.as_mut_ptr(),
                scales.as_mut_ptr(),
                dequant.as_mut_ptr(),
                1,
            )
        };
        assert_eq!(rc, 0, "kiln_w4a16_quantize_and_pack_host failed with status {rc}");
        (packed, scales.into_iter().map(f16::from_bits).collect(), dequant)
    }
}
