// Links against libtei_b200.so, which is built by `python text-embeddings-inference_b200/build.py`
// (nvcc, sm_100a).  TEI_B200_LIB_DIR points at the directory that holds it.
fn main() {
    println!("cargo:rerun-if-env-changed=TEI_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("TEI_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=tei_b200");
}
