// Links libdyninfer_cuda.so. DYNINFER_CUDA_LIB_DIR names the directory that holds it (the
// in-tree build leaves it in dyninfer_b200/).
fn main() {
    println!("cargo:rerun-if-env-changed=DYNINFER_CUDA_LIB_DIR");
    if let Ok(dir) = std::env::var("DYNINFER_CUDA_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=dyninfer_cuda");
}
