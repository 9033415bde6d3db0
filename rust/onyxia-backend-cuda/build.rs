//! Links `libonyxia_cuda.so` (and, through its run path, `libonyxia_ir.so`).
//!
//! `ONYXIA_CUDA_DIR` names the checkout of the native sources (the directory that holds
//! `onyxia_b200/` and `include/`). With the `build-native` feature the libraries are built
//! there first — the same two compiler invocations `python -m onyxia_b200.build` runs:
//! g++ for the host IR, nvcc `-gencode arch=compute_100a,code=sm_100a` for the backend.
use std::env;
use std::path::PathBuf;
use std::process::Command;

fn main() {
    println!("cargo:rerun-if-env-changed=ONYXIA_CUDA_DIR");
    let root = PathBuf::from(env::var("ONYXIA_CUDA_DIR").expect("set ONYXIA_CUDA_DIR to the native checkout"));
    let lib_dir = root.join("onyxia_b200");
    if env::var_os("CARGO_FEATURE_BUILD_NATIVE").is_some() {
        let status = Command::new(env::var("PYTHON").unwrap_or_else(|_| "python3".into()))
            .args(["-m", "onyxia_b200.build"])
            .current_dir(&root)
            .status()
            .expect("cannot start the native build");
        assert!(status.success(), "the native build failed");
    }
    assert!(lib_dir.join("libonyxia_cuda.so").exists(), "libonyxia_cuda.so not found under {}", lib_dir.display());
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=onyxia_cuda");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", lib_dir.display());
    println!("cargo:include={}", root.join("include").display());
}
