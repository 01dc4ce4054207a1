// Tells cargo where liblisa_cuda.so lives: LISA_CUDA_LIB_DIR, else ../../lisa_b200/lib beside this crate.
fn main() {
    let dir = std::env::var("LISA_CUDA_LIB_DIR").unwrap_or_else(|_| {
        let here = std::path::PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").unwrap());
        here.join("../../lisa_b200/lib").to_string_lossy().into_owned()
    });
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=lisa_cuda");
    println!("cargo:rerun-if-env-changed=LISA_CUDA_LIB_DIR");
}
