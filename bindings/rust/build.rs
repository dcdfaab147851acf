// Links the façade against librstorch_b200.so.  RSTORCH_B200_LIB_DIR names the folder
// that holds the library (the output folder of `python -m rstorch_b200.build`).
fn main() {
    println!("cargo:rerun-if-env-changed=RSTORCH_B200_LIB_DIR");
    if let Ok(dir) = std::env::var("RSTORCH_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
        println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
    }
    println!("cargo:rustc-link-lib=dylib=rstorch_b200");
}
