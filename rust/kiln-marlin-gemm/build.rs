// Compiles the CUDA sources of kiln_b200/csrc for sm_100a only and links them into the crate.
// Stands where kiln's crates/kiln-marlin-gemm/build.rs stands (arch list 80;86;89;90 there).
use std::env;
use std::path::PathBuf;

fn main() {
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    let csrc = manifest.join("../../kiln_b200/csrc");
    let cuda_root = env::var("CUDA_HOME")
        .or_else(|_| env::var("CUDA_ROOT"))
        .unwrap_or_else(|_| "/usr/local/cuda".to_string());

    let mut build = cc::Build::new();
    build.cuda(true).cpp(true);
    build.include(&csrc).include(manifest.join("../../include"));
    build.include(format!("{cuda_root}/include"));
    for flag in ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr"] {
        build.flag(flag);
    }
    build.flag("-Xcompiler").flag("-fPIC");
    // tcgen05 / TMEM need the architecture-specific target
    build.flag("-gencode=arch=compute_100a,code=sm_100a");
    for f in [
        "api.cu",
        "decode_w4a16.cu",
        "epilogue_w4a16.cu",
        "prefill_w4a16_umma.cu",
        "repack.cu",
    ] {
        build.file(csrc.join(f));
    }
    build.compile("kiln_w4a16");

    println!("cargo:rustc-link-search=native={cuda_root}/lib64");
    println!("cargo:rustc-link-lib=cudart");
    println!("cargo:rerun-if-changed=../../kiln_b200/csrc/");
    println!("cargo:rerun-if-changed=../../include/kiln_w4a16.h");
}
