// Points the linker at libggr_attn.so. GGR_ATTN_LIB_DIR names the directory that holds it (the package
// directory of the Python build, or wherever the library was installed).
fn main() {
    println!("cargo:rerun-if-env-changed=GGR_ATTN_LIB_DIR");
    if let Ok(dir) = std::env::var("GGR_ATTN_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=ggr_attn");
}
