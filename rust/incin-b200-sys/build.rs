// Links the two shared libraries that `python -m incin_b200 build` (or `make -C csrc`) leaves in incin_b200/lib.
// INCIN_B200_LIB_DIR overrides the search path.
use std::env;
use std::path::PathBuf;

fn main() {
    let dir = env::var("INCIN_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|_| {
        PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap()).join("../../incin_b200/lib")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=incin_sm100");
    println!("cargo:rustc-link-lib=dylib=incin_host");
    println!("cargo:rerun-if-env-changed=INCIN_B200_LIB_DIR");
}
