// Builds libssd_b200.so from the CUDA sources with nvcc for sm_100a and tells cargo how to link it.
//
// Same role as the link-argument script of the reference's crates (trading_bots/build.rs:1-19, which only emits rpath and
// -ltorch/-lc10) plus the compile step the vendored torch-sys does with cc::Build for its C++ shim
// (vendor/torch-sys-0.25.0/build.rs:403-428); nvcc is driven directly because cc has no notion of -gencode.
//
// Environment:
//   SSD_B200_SRC   root of this repository's checkout (default: two levels above this crate)
//   NVCC           nvcc binary (default: nvcc on PATH, then /usr/local/cuda/bin/nvcc)
//   SSD_B200_LIB_DIR  if set, skip the build and link the libssd_b200.so found there
use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

const SOURCES: [&str; 7] = [
    "ssd_api.cu",
    "ssd_simt.cu",
    "ssd_decode.cu",
    "ssd_tensor.cu",
    "ssd_noalloc.cu",
    "ssd_prepost.cu",
    "ssd_sp.cu",
];

fn nvcc() -> String {
    if let Ok(p) = env::var("NVCC") {
        return p;
    }
    if Command::new("nvcc").arg("--version").output().is_ok() {
        return "nvcc".to_string();
    }
    "/usr/local/cuda/bin/nvcc".to_string()
}

fn main() {
    let os = env::var("CARGO_CFG_TARGET_OS").expect("Unable to get TARGET_OS");
    if os != "linux" {
        panic!("ssd-sys targets linux + CUDA (sm_100a) only");
    }
    let manifest = PathBuf::from(env::var("CARGO_MANIFEST_DIR").unwrap());
    let root = env::var("SSD_B200_SRC")
        .map(PathBuf::from)
        .unwrap_or_else(|_| manifest.join("..").join(".."));
    let csrc = root.join("trading_bot_0_b200").join("csrc");
    let header = root.join("include").join("ssd_b200.h");
    println!("cargo:rerun-if-changed=build.rs");
    println!("cargo:rerun-if-changed={}", header.display());
    println!("cargo:rerun-if-env-changed=SSD_B200_LIB_DIR");

    let lib_dir: PathBuf = match env::var_os("SSD_B200_LIB_DIR") {
        Some(d) => PathBuf::from(d),
        None => {
            let out = PathBuf::from(env::var("OUT_DIR").unwrap());
            build_library(&csrc, &out);
            out
        }
    };
    println!("cargo:rustc-link-search=native={}", lib_dir.display());
    println!("cargo:rustc-link-lib=dylib=ssd_b200");
    println!("cargo:rustc-link-arg=-Wl,-rpath={}", lib_dir.display());
    // dependants find the directory as DEP_SSD_B200_LIB_DIR (the `links` key), the way torch-sys hands out
    // DEP_TCH_LIBTORCH_LIB
    println!("cargo:lib_dir={}", lib_dir.display());
    println!("cargo:include={}", root.join("include").display());
}

fn build_library(csrc: &Path, out: &Path) {
    let mut objects = Vec::new();
    for src in SOURCES {
        let path = csrc.join(src);
        println!("cargo:rerun-if-changed={}", path.display());
        let obj = out.join(format!("{src}.o"));
        let status = Command::new(nvcc())
            .args(["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"])
            .args(["-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-c"])
            .arg(&path)
            .arg("-o")
            .arg(&obj)
            .status()
            .expect("failed to run nvcc");
        assert!(status.success(), "nvcc failed on {}", path.display());
        objects.push(obj);
    }
    for h in ["common.cuh", "umma.cuh", "ssd_internal.h"] {
        println!("cargo:rerun-if-changed={}", csrc.join(h).display());
    }
    let status = Command::new(nvcc())
        .args(["-shared", "-Xcompiler", "-fPIC"])
        .args(&objects)
        .arg("-o")
        .arg(out.join("libssd_b200.so"))
        .arg("-ldl")
        .status()
        .expect("failed to run nvcc (link)");
    assert!(status.success(), "linking libssd_b200.so failed");
}
