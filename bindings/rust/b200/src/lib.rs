//! B200 back end for bullet's trainer, written against bullet's own crates.  SOURCE ONLY in the
//! repository that ships it: no Rust toolchain is available there, so this crate has never been
//! compiled; `tests/test_host.py` checks that every `b200_*` symbol used here is declared by
//! `include/bullet_b200.h`.
//!
//! Where it plugs in.  `bullet_trainer::run::train` is generic over `G: Gpu` and enters the device
//! through `Function::execute`, `Optimiser::update` and `PreparedBatchHost::copy_to_device_async`
//! (crates/trainer/src/run.rs:75-250).  This crate replaces those three for the recognised family of
//! graphs: `recognise` turns `ModelDefinition.ir()` into a `b200_net_desc`, `B200Trainer` owns the
//! library handle, `train_b200` is the loop.  Two stanzas make the existing examples take this path:
//!
//! ```toml
//! # crates/trainer/Cargo.toml                      # crates/bullet_lib/Cargo.toml
//! [features]                                       [features]
//! b200 = ["dep:b200"]                              b200 = ["bullet_trainer/b200"]
//! [dependencies]
//! b200 = { path = "../b200", optional = true }
//! ```
//!
//! and in crates/bullet_lib/src/value.rs the `run` method (value.rs:119-211) calls, under
//! `#[cfg(feature = "b200")]`, `b200::B200Trainer::new(self.optimiser.definition(), 0, block_rows,
//! batch_size)`, copies every weight across with `load_weight_from_host`, and hands `train_b200` the same
//! schedule, loader and callbacks it hands `train` today; a graph that is not recognised ends the run
//! with the recogniser's message (there is no fallback to the generic path inside one run).
pub mod recognise;
pub mod train;

pub use recognise::{Recognised, recognise};
pub use train::{B200Error, B200Trainer, train_b200};
