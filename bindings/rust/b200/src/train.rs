//! The training loop of crates/trainer/src/run.rs:75-250 on the C ABI of libbullet_b200.so.
//!
//! `B200Trainer` stands where `Optimiser<G, O>` stands in the reference (weights by id, per-weight
//! AdamW parameters, checkpoints); `train_b200` is `train`: a loader thread feeds prepared batches
//! through a bounded channel, the training thread enqueues one step, hands the NEXT batch to the
//! library while the GPU computes (the library packs it into pinned memory and copies it on its own
//! stream: run/dataloader.rs:41-61 without the staging sync), then reads the step's loss and calls
//! the callbacks with `loss / batch_size`, exactly as run.rs:212-247 does.
use std::{
    collections::BTreeMap,
    ffi::{CStr, CString},
    ptr,
    sync::mpsc,
    thread,
    time::Instant,
};

use b200_sys::*;
use bullet_compiler::tensor::TValue;
use bullet_trainer::{
    model::ModelDefinition,
    optimiser::adam::AdamWParams,
    run::{DataLoader, DataLoadingError, PreparedBatchHost, Step, TrainingSchedule, logger},
};

use crate::recognise::{Recognised, recognise};

#[derive(Debug)]
pub enum B200Error {
    /// the graph is outside the family the library runs; the message says why
    Unrecognised(String),
    /// an entry point returned a negative status; the message is `b200_last_error()`
    Library { code: i32, message: String },
    DataLoading(DataLoadingError),
    /// a batch misses an input the graph names, or holds the wrong type or size
    Batch(String),
}

fn check(code: i32) -> Result<(), B200Error> {
    if code >= 0 {
        return Ok(());
    }
    let message = unsafe { CStr::from_ptr(b200_last_error()) }.to_string_lossy().into_owned();
    Err(B200Error::Library { code, message })
}

pub struct B200Trainer {
    net: *mut b200_net,
    recognised: Recognised,
    batch_size: usize,
}

// one training thread drives the handle (the C ABI allows a second thread only for uploads)
unsafe impl Send for B200Trainer {}

impl Drop for B200Trainer {
    fn drop(&mut self) {
        unsafe { b200_net_destroy(self.net) };
    }
}

impl B200Trainer {
    /// `Function::new` + `prealloc` + `Optimiser::new` (crates/gpu/src/function.rs:73,180,
    /// crates/trainer/src/optimiser.rs:98-133): recognise the graph, allocate everything once.
    pub fn new(defn: &ModelDefinition, device: i32, ft_block_rows: usize, batch_size: usize) -> Result<Self, B200Error> {
        let recognised = recognise(defn, ft_block_rows, batch_size).map_err(B200Error::Unrecognised)?;
        let mut net = ptr::null_mut();
        check(unsafe { b200_net_create(device, ptr::null_mut(), &recognised.desc, &mut net) })?;
        Ok(Self { net, recognised, batch_size })
    }

    pub fn recognised(&self) -> &Recognised {
        &self.recognised
    }

    fn abi_name(&self, id: &str) -> Result<CString, B200Error> {
        self.recognised
            .weights
            .iter()
            .find(|(graph_id, _)| graph_id == id)
            .map(|(_, abi)| CString::new(*abi).unwrap())
            .ok_or_else(|| B200Error::Batch(format!("no weight with id '{id}'")))
    }

    /// Optimiser::load_weights_from_host (optimiser.rs:208-212), one weight at a time.
    pub fn load_weight_from_host(&mut self, id: &str, values: &[f32]) -> Result<(), B200Error> {
        let name = self.abi_name(id)?;
        check(unsafe { b200_net_set_tensor(self.net, name.as_ptr(), B200_KIND_WEIGHT, values.as_ptr(), values.len() as i64) })
    }

    /// Buffer::to_host of one weight (optimiser.rs:214-216).
    pub fn weight_to_host(&self, id: &str) -> Result<Vec<f32>, B200Error> {
        let name = self.abi_name(id)?;
        let mut n = 0i64;
        check(unsafe { b200_net_tensor_size(self.net, name.as_ptr(), &mut n) })?;
        let mut out = vec![0.0f32; n as usize];
        check(unsafe { b200_net_get_tensor(self.net, name.as_ptr(), B200_KIND_WEIGHT, out.as_mut_ptr(), n) })?;
        Ok(out)
    }

    /// Optimiser::set_params_for_weight (optimiser.rs:204-206).
    pub fn set_params_for_weight(&mut self, id: &str, params: AdamWParams) -> Result<(), B200Error> {
        let name = self.abi_name(id)?;
        let p = b200_adamw_params {
            decay: params.decay,
            beta1: params.beta1,
            beta2: params.beta2,
            min_weight: params.min_weight,
            max_weight: params.max_weight,
        };
        check(unsafe { b200_net_set_adamw(self.net, name.as_ptr(), &p) })
    }

    /// Optimiser::write_to_checkpoint / load_from_checkpoint (optimiser.rs:218-236): the same three files.
    pub fn write_to_checkpoint(&self, path: &str) -> Result<(), B200Error> {
        let dir = CString::new(path).unwrap();
        check(unsafe { b200_checkpoint_save(self.net, dir.as_ptr()) })
    }

    pub fn load_from_checkpoint(&mut self, path: &str) -> Result<(), B200Error> {
        let dir = CString::new(path).unwrap();
        check(unsafe { b200_checkpoint_load(self.net, dir.as_ptr()) })
    }

    /// PreparedBatchHost::copy_to_device_async (run/dataloader.rs:41-61) into staging slot `slot`.
    fn upload(&mut self, slot: i32, batch: &PreparedBatchHost) -> Result<(), B200Error> {
        let r = &self.recognised;
        let ints = |inputs: &BTreeMap<String, TValue>, name: &str| -> Result<*const i32, B200Error> {
            match inputs.get(name) {
                Some(TValue::I32(v)) => Ok(v.as_ptr()),
                _ => Err(B200Error::Batch(format!("batch has no i32 input '{name}'"))),
            }
        };
        let stm = ints(&batch.inputs, &r.stm)?;
        let ntm = ints(&batch.inputs, &r.ntm)?;
        let buckets = match &r.buckets {
            Some(name) => ints(&batch.inputs, name)?,
            None => ptr::null(),
        };
        let Some(TValue::F32(targets)) = batch.inputs.get(&r.targets) else {
            return Err(B200Error::Batch(format!("batch has no f32 input '{}'", r.targets)));
        };
        if targets.len() > self.batch_size {
            return Err(B200Error::Batch(format!("{} positions in a batch of at most {}", targets.len(), self.batch_size)));
        }
        check(unsafe { b200_batch_upload(self.net, slot, stm, ntm, buckets, targets.as_ptr(), targets.len() as i32) })
    }
}

/// `train` (crates/trainer/src/run.rs:75-81) for the B200 library: same schedule, same loader trait,
/// same callbacks (they receive the trainer where the reference passes the optimiser).
pub fn train_b200(
    trainer: &mut B200Trainer,
    schedule: TrainingSchedule,
    dataloader: impl DataLoader,
    mut batch_callback: impl FnMut(&mut B200Trainer, Step, f32),
    mut superbatch_callback: impl FnMut(&mut B200Trainer, Step),
) -> Result<(), B200Error> {
    let timer = Instant::now();
    logger::clear_colours();
    println!("{}", logger::ansi("Training on NVIDIA B200 (bullet_b200)", "34;1"));

    let steps = schedule.steps;
    let (sender, receiver) = mpsc::sync_channel::<PreparedBatchHost>(32);
    let loader = thread::spawn(move || {
        let mut step = Step::from(steps);
        dataloader.map_batches(step, steps.batch_size, |batch| {
            sender.send(batch).unwrap();
            step.step();
            step.finished()
        })
    });

    let grad_factor = 1.0 / steps.batch_size as f32; // run.rs:130-131
    let first = receiver.recv().map_err(|_| B200Error::DataLoading(DataLoadingError::NoBatchesReceived))?;
    let mut slot = 0i32;
    trainer.upload(slot, &first)?;
    drop(first);

    let lr = schedule.lr_schedule;
    let mut batch_queued = true;
    let mut step = Step::from(steps);
    let mut prev_lr = lr(step);
    let mut superbatch_timer = Instant::now();
    let mut running_loss = 0.0;
    let mut superbatch_positions = 0;

    while batch_queued {
        if step.finished() {
            return Err(B200Error::DataLoading(DataLoadingError::TooManyBatchesReceived));
        }
        let lrate = lr(step);
        if step.batch() == 0 {
            if lrate < prev_lr {
                println!("LR dropped to {}", logger::ansi(lrate, logger::num_cs()));
            } else if lrate > prev_lr {
                println!("LR increased to {}", logger::ansi(lrate, logger::num_cs()));
            }
        }
        prev_lr = lrate;

        // backward graph + optimiser update (run.rs:185-192): only enqueues
        check(unsafe { b200_step(trainer.net, slot, lrate, grad_factor) })?;

        // the next batch goes to another slot while this step runs (run.rs:194-204)
        if let Ok(next) = receiver.recv() {
            let next_slot = (slot + 1) % B200_NUM_SLOTS;
            trainer.upload(next_slot, &next)?;
            slot = next_slot;
        } else {
            batch_queued = false;
        }

        // run.rs:206-221: wait for the step, read the loss
        let mut loss = 0.0f32;
        check(unsafe { b200_loss(trainer.net, &mut loss) })?;
        let error = loss / steps.batch_size as f32;
        running_loss += error;
        superbatch_positions += steps.batch_size;

        if step.batch().is_multiple_of(schedule.log_rate) {
            logger::report_superbatch_progress(step, &superbatch_timer, superbatch_positions);
        }
        batch_callback(trainer, step, error);

        if step.batch() == step.batches_per_superbatch() - 1 {
            let error = running_loss / steps.batches_per_superbatch as f32;
            running_loss = 0.0;
            let total_time = timer.elapsed().as_secs_f32();
            let sb_time = superbatch_timer.elapsed().as_secs_f32();
            let sb = step.superbatch();
            logger::report_superbatch_finished(sb, error, sb_time, total_time, superbatch_positions);
            logger::report_time_left(steps, sb, total_time);
            superbatch_callback(trainer, step);
            superbatch_positions = 0;
            superbatch_timer = Instant::now();
        }
        step.step();
    }

    check(unsafe { b200_sync(trainer.net) })?;
    loader.join().unwrap().map_err(B200Error::DataLoading)?;
    Ok(())
}
