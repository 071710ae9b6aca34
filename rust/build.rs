// Links libakasha_b200.so. AKASHA_B200_LIB_DIR names the directory that holds it
// (akasha-core_b200/ after `python akasha-core_b200/build.py`).
fn main() {
    let dir = std::env::var("AKASHA_B200_LIB_DIR").unwrap_or_else(|_| "../akasha-core_b200".to_string());
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=akasha_b200");
    println!("cargo:rerun-if-env-changed=AKASHA_B200_LIB_DIR");
}
