// Links libpm_b200.so (built by `python photon-mamba2-llm_b200/build.py`) and the CUDA runtime.
// PM_B200_LIB_DIR = directory that holds libpm_b200.so; CUDA_HOME defaults to /usr/local/cuda.
fn main() {
    let lib_dir = std::env::var("PM_B200_LIB_DIR").expect("set PM_B200_LIB_DIR to the directory of libpm_b200.so");
    let cuda = std::env::var("CUDA_HOME").unwrap_or_else(|_| "/usr/local/cuda".into());
    println!("cargo:rustc-link-search=native={lib_dir}");
    println!("cargo:rustc-link-search=native={cuda}/lib64");
    println!("cargo:rustc-link-lib=dylib=pm_b200");
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rerun-if-env-changed=PM_B200_LIB_DIR");
}
