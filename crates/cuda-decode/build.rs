// Links libcuda_decode.so, built by `make -C rustane_b200/csrc` (nvcc, sm_100a only).
// CUDA_DECODE_LIB_DIR names the directory that holds it; the default is the package directory
// of this repository.  Source only: never compiled here (no Rust toolchain in the build image).
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("CUDA_DECODE_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../rustane_b200")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=cuda_decode");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=CUDA_DECODE_LIB_DIR");
}
