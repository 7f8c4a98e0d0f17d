// Links libblum.so from the directory it is built in (python -m luminal_b200.build), or from BLUM_LIB_DIR.
fn main() {
    let dir = std::env::var("BLUM_LIB_DIR").unwrap_or_else(|_| {
        let here = std::path::PathBuf::from(std::env::var("CARGO_MANIFEST_DIR").unwrap());
        here.parent().unwrap().to_string_lossy().into_owned()
    });
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=blum");
    println!("cargo:rerun-if-env-changed=BLUM_LIB_DIR");
}
