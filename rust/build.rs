// Build hook for xn-core's `cuda` feature.  UNCOMPILED here (no Rust toolchain on the machine this was written
// on).  Today xn-core/build.rs:9-15 compiles cuda-kernels/*.cu to PTX strings; the tcgen05 / TMA kernels need
// host-side descriptor set-up, so this path builds a shared library with nvcc for sm_100a and links it.
// Expects the engine's sources under `xn_mm/` next to Cargo.toml (a copy or a submodule of this repository:
// `xn_mm/xn_b200/csrc/*.cu`, `xn_mm/include/xn_mm.h`).
use std::path::PathBuf;
use std::process::Command;

fn main() {
    if std::env::var("CARGO_FEATURE_CUDA").is_err() {
        return;
    }
    let out = PathBuf::from(std::env::var("OUT_DIR").unwrap());
    let csrc = PathBuf::from("xn_mm/xn_b200/csrc");
    println!("cargo:rerun-if-changed=xn_mm/include/xn_mm.h");
    let mut sources = Vec::new();
    for entry in std::fs::read_dir(&csrc).expect("xn_mm/xn_b200/csrc is missing") {
        let path = entry.unwrap().path();
        println!("cargo:rerun-if-changed={}", path.display());
        if path.extension().map(|e| e == "cu").unwrap_or(false) {
            sources.push(path);
        }
    }
    sources.sort();
    let nvcc = std::env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    let mut cmd = Command::new(nvcc);
    cmd.args([
        "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
        "-Xcompiler", "-fPIC", "-shared", "-o",
    ])
    .arg(out.join("libxn_mm.so"))
    .args(&sources)
    .arg("-lcuda");
    let status = cmd.status().expect("failed to run nvcc");
    assert!(status.success(), "nvcc failed building libxn_mm.so");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=xn_mm");
}
