// Links librunit_cuda.so.  RUNIT_CUDA_LIB_DIR points at the directory that holds it (the in-tree build
// leaves it in runit_mac_b200/); the role of METALLIB_PATH in crates/kernels/build.rs:13-22.
fn main() {
    let dir = std::env::var("RUNIT_CUDA_LIB_DIR").unwrap_or_else(|_| "../../runit_mac_b200".to_string());
    println!("cargo:rustc-link-search=native={}", dir);
    println!("cargo:rustc-link-lib=dylib=runit_cuda");
    println!("cargo:rerun-if-env-changed=RUNIT_CUDA_LIB_DIR");
}
