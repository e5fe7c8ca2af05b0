// Points the linker at libbullet_b200.so.  Set B200_LIB_DIR to the directory that holds it
// (in this repository: bullet_b200/, after `python -m bullet_b200.build`).
fn main() {
    let dir = std::env::var("B200_LIB_DIR").expect("set B200_LIB_DIR to the directory of libbullet_b200.so");
    println!("cargo:rustc-link-search=native={dir}");
    println!("cargo:rustc-link-lib=dylib=bullet_b200");
    println!("cargo:rerun-if-env-changed=B200_LIB_DIR");
}
