// Links the prebuilt kernel library.  CATENA_B200_LIB_DIR points at the directory that holds
// libcatena_b200.so (the `catena-lang_b200/` directory of the kernel repository).
fn main() {
    if let Ok(dir) = std::env::var("CATENA_B200_LIB_DIR") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=catena_b200");
    println!("cargo:rerun-if-env-changed=CATENA_B200_LIB_DIR");
}
