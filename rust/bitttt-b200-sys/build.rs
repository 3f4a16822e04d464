// Links libbitttt_b200.so.  BITTTT_B200_LIB_DIR names the directory that holds it (the in-tree
// build puts it into bit-ttt-engine_b200/lib/); the CUDA runtime is linked by the library itself.
use std::env;
use std::path::PathBuf;

fn main() {
    println!("cargo:rerun-if-env-changed=BITTTT_B200_LIB_DIR");
    let dir = env::var("BITTTT_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        // default: the repository layout, this crate sitting in rust/bitttt-b200-sys
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../bit-ttt-engine_b200/lib")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=bitttt_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", dir.display());
}
