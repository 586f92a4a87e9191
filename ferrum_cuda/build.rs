//! Points the linker at libferrum_cuda.so. The library is built outside cargo, by nvcc
//! (`python -m ferrum_cpu_b200.build`, or the Makefile rule of your choice running
//! `nvcc -gencode arch=compute_100a,code=sm_100a -O3 -shared -Xcompiler -fPIC csrc/*.cu csrc/*.cpp`);
//! FERRUM_CUDA_LIB_DIR names the directory that holds it.
fn main() {
    println!("cargo:rerun-if-env-changed=FERRUM_CUDA_LIB_DIR");
    let dir = std::env::var("FERRUM_CUDA_LIB_DIR")
        .expect("set FERRUM_CUDA_LIB_DIR to the directory that holds libferrum_cuda.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=ferrum_cuda");
    // the library links the CUDA runtime statically; only the driver is needed at run time
    println!("cargo:rustc-link-arg=-Wl,-rpath,{dir}");
}
