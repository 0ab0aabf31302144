// Points rustc at libb200q.so.  B200Q_LIB_DIR is the directory that holds the library
// (`python -m boostr_b200.build` writes it to boostr_b200/libb200q.so).
fn main() {
    if let Ok(dir) = std::env::var("B200Q_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=b200q");
    println!("cargo:rerun-if-env-changed=B200Q_LIB_DIR");
}
