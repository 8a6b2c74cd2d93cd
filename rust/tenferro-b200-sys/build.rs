// Tells rustc where libtenferro_b200.so lives: TENFERRO_B200_LIB_DIR, else the in-tree build
// directory of this repository (tenferro-rs_b200/lib, made by `make -C tenferro-rs_b200/csrc`).
use std::env;
use std::path::PathBuf;

fn main() {
    println!("cargo:rerun-if-env-changed=TENFERRO_B200_LIB_DIR");
    let dir = env::var_os("TENFERRO_B200_LIB_DIR").map(PathBuf::from).unwrap_or_else(|| {
        PathBuf::from(env::var_os("CARGO_MANIFEST_DIR").expect("cargo sets CARGO_MANIFEST_DIR"))
            .join("../../tenferro-rs_b200/lib")
    });
    println!("cargo:rustc-link-search=native={}", dir.display());
    println!("cargo:rustc-link-lib=dylib=tenferro_b200");
}
