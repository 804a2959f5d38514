//! Links `libneura_cuda.so`.  `NEURA_CUDA_LIB_DIR` names the directory that holds it (the library is built from
//! `neura_b200/csrc` with `python -m neura_b200.build`; it needs nvcc and targets sm_100a only).
fn main() {
    if let Ok(dir) = std::env::var("NEURA_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=neura_cuda");
    println!("cargo:rerun-if-env-changed=NEURA_CUDA_LIB_DIR");
}
