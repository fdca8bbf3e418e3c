// Points the linker at libtlb200.so (built by `python -m tl_b200.build` from the CUDA sources of this repository).
// TLB200_LIB_DIR names the directory holding it; the run-time search path is set to the same place.
fn main() {
    let dir = std::env::var("TLB200_LIB_DIR").unwrap_or_else(|_| "../../".to_string());
    println!("cargo:rustc-link-search=native={}", dir);
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir);
    println!("cargo:rerun-if-env-changed=TLB200_LIB_DIR");
}
