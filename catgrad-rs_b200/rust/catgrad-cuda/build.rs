// NOT compiled here (no Rust toolchain): source only.
fn main() {
    let dir = std::env::var("CATGRAD_CUDA_LIB_DIR").expect("set CATGRAD_CUDA_LIB_DIR to the directory of libcatgrad_cuda.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=catgrad_cuda");
}
