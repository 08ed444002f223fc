// Points the linker at libellm_attn.so (built by `python -m ellm_b200.build`).
// ELLM_ATTN_LIB_DIR = the directory that holds it; default: ../../ellm_b200 relative to this crate.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("ELLM_ATTN_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../ellm_b200")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=ellm_attn");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
    println!("cargo:rerun-if-env-changed=ELLM_ATTN_LIB_DIR");
}
