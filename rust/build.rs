//! Build step of the CUDA backend for the MoE path: compiles the hand-written kernels under
//! `maxuna_b200/csrc/` for sm_100a with nvcc into a static archive and links it, together with the CUDA
//! runtime, into the `laguna` binary.  Goes next to the reference's Cargo.toml (as `build.rs`), with
//! `LMOE_CSRC` pointing at the kernel sources when they are not vendored under `cuda/`.
//!
//! There is no fallback: without nvcc the build fails, and without a CUDA device every op of
//! `ops::cuda` returns an error (`LMOE_ERR_CUDA`).
//!
//! NOT COMPILED in the environment this file was written in (no Rust toolchain there); it is the text a
//! maintainer adds.  The nvcc command line is the one the Python build of the same sources uses.
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

fn main() {
    let out_dir = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    let csrc = env::var("LMOE_CSRC").map(PathBuf::from).unwrap_or_else(|_| PathBuf::from("cuda/csrc"));
    let include = env::var("LMOE_INCLUDE").map(PathBuf::from).unwrap_or_else(|_| PathBuf::from("cuda/include"));
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    let cuda_home = env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".to_string());

    println!("cargo:rerun-if-env-changed=LMOE_CSRC");
    println!("cargo:rerun-if-env-changed=NVCC");
    println!("cargo:rerun-if-changed={}", include.join("lmoe.h").display());

    let mut objects = Vec::new();
    let mut sources: Vec<PathBuf> = std::fs::read_dir(&csrc)
        .unwrap_or_else(|e| panic!("kernel sources not found at {}: {e}", csrc.display()))
        .filter_map(|e| e.ok().map(|e| e.path()))
        .filter(|p| p.extension().map(|x| x == "cu").unwrap_or(false))
        .collect();
    sources.sort();
    assert!(!sources.is_empty(), "no .cu files under {}", csrc.display());
    for src in &sources {
        println!("cargo:rerun-if-changed={}", src.display());
        let obj = out_dir.join(Path::new(src.file_name().unwrap()).with_extension("o"));
        // sm_100a only: the kernels use tcgen05 / TMEM / bulk-tensor copies and have no other target
        let status = Command::new(&nvcc)
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
            .args(["-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"])
            .arg("-I").arg(&include)
            .arg("-c").arg(src)
            .arg("-o").arg(&obj)
            .status()
            .unwrap_or_else(|e| panic!("could not run {nvcc}: {e}"));
        assert!(status.success(), "nvcc failed on {}", src.display());
        objects.push(obj);
    }
    for h in std::fs::read_dir(&csrc).unwrap().filter_map(|e| e.ok()) {
        if h.path().extension().map(|x| x == "cuh").unwrap_or(false) {
            println!("cargo:rerun-if-changed={}", h.path().display());
        }
    }
    let archive = out_dir.join("liblmoe.a");
    let _ = std::fs::remove_file(&archive);
    let status = Command::new("ar").arg("crs").arg(&archive).args(&objects).status().expect("ar");
    assert!(status.success(), "ar failed");

    println!("cargo:rustc-link-search=native={}", out_dir.display());
    println!("cargo:rustc-link-lib=static=lmoe");
    println!("cargo:rustc-link-search=native={cuda_home}/lib64");
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rustc-link-lib=dylib=stdc++");
}
