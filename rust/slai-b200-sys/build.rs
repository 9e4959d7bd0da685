// Links against libslai_b200.so built by `python -m slai_b200.build`.
// Source only: this repository's environment has no Rust toolchain, the C ABI is the tested boundary.
fn main() {
    let dir = std::env::var("SLAI_B200_LIB_DIR").unwrap_or_else(|_| "../../slai_b200".to_string());
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=slai_b200");
    println!("cargo:rerun-if-env-changed=SLAI_B200_LIB_DIR");
}
