//! Raw declarations of `include/bullet_b200.h`, one to one.  Not compiled in the repository
//! that ships it (no Rust toolchain there); `tests/test_host.py` checks that every symbol of
//! the header is declared here.
#![allow(non_camel_case_types)]
use std::os::raw::{c_char, c_int, c_void};

pub const B200_OK: c_int = 0;
pub const B200_ERR_ARG: c_int = -1;
pub const B200_ERR_STATE: c_int = -2;
pub const B200_ERR_CUDA: c_int = -3;
pub const B200_ERR_DATA: c_int = -4;
pub const B200_ERR_UNSUPPORTED: c_int = -5;

pub const B200_ACT_NONE: i32 = 0;
pub const B200_ACT_CRELU: i32 = 1;
pub const B200_ACT_SCRELU: i32 = 2;

pub const B200_KIND_WEIGHT: c_int = 0;
pub const B200_KIND_MOMENTUM: c_int = 1;
pub const B200_KIND_VELOCITY: c_int = 2;
pub const B200_KIND_GRAD: c_int = 3;

pub const B200_GAME_CHESS768: i32 = 0;
pub const B200_GAME_CHESS_BUCKETS_MIRRORED: i32 = 1;
pub const B200_GAME_ATAXX147: i32 = 2;

pub const B200_QUANT_FLOAT: i32 = 0;
pub const B200_QUANT_I8: i32 = 1;
pub const B200_QUANT_I16: i32 = 2;
pub const B200_QUANT_I32: i32 = 3;

pub const B200_NUM_SLOTS: c_int = 3;
pub const B200_EXCHANGE_HANDLE_BYTES: usize = 192;
pub const B200_OP_NOALLOC_MAX_POSITIONS: i32 = 16384;

#[repr(C)]
pub struct b200_net {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct b200_net_desc {
    pub n_inputs: i32,
    pub nnz: i32,
    pub ft_out: i32,
    pub ft_act: i32,
    pub pairwise: i32,
    pub factoriser_rows: i32,
    pub n_out_buckets: i32,
    pub n_dense: i32,
    pub dense_out: [i32; 3],
    pub dense_act: [i32; 3],
    pub ft_block_rows: i32,
    pub max_batch: i32,
}

pub const B200_OPT_ADAMW: i32 = 0;
pub const B200_OPT_RADAM: i32 = 1;
pub const B200_OPT_RANGER: i32 = 2;
pub const B200_KIND_SLOW: c_int = 4;

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct b200_optimiser_params {
    pub kind: i32,
    pub decay: f32,
    pub beta1: f32,
    pub beta2: f32,
    pub min_weight: f32,
    pub max_weight: f32,
    pub n_sma_threshold: f32,
    pub alpha: f32,
    pub k: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct b200_adamw_params {
    pub decay: f32,
    pub beta1: f32,
    pub beta2: f32,
    pub min_weight: f32,
    pub max_weight: f32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct b200_timings {
    pub ft_forward: f32,
    pub dense_forward: f32,
    pub dense_backward: f32,
    pub ft_backward: f32,
    pub factoriser_grad: f32,
    pub optimiser: f32,
    pub total: f32,
    pub steps: i32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct b200_ft_op {
    pub n_inputs: i32,
    pub nnz: i32,
    pub ft_out: i32,
    pub ft_act: i32,
    pub pairwise: i32,
    pub ft_block_rows: i32,
    pub n: i32,
    pub table: *const f32,
    pub bias: *const f32,
    pub idx_stm: *const u16,
    pub idx_nstm: *const u16,
    pub x: *mut f32,
    pub u: *mut f32,
}

/// One entry of an export in the reference's `SavedFormat` scheme
/// (crates/trainer/src/model/weights.rs:183-335): custom bytes when `id` is null, else a weight
/// with the built-in transforms and a quantisation target.
#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct b200_saved_format {
    pub id: *const c_char,
    pub custom: *const c_void,
    pub custom_len: i64,
    pub quant: i32,
    pub multiplier: i32,
    pub round: i32,
    pub transpose: i32,
    pub merge_factoriser: i32,
}

extern "C" {
    pub fn b200_last_error() -> *const c_char;
    pub fn b200_version() -> c_int;

    pub fn b200_net_create(device: c_int, stream: *mut c_void, desc: *const b200_net_desc, out: *mut *mut b200_net) -> c_int;
    pub fn b200_net_destroy(net: *mut b200_net) -> c_int;
    pub fn b200_net_set_option(net: *mut b200_net, key: *const c_char, value: i64) -> c_int;
    pub fn b200_net_tensor_size(net: *mut b200_net, name: *const c_char, n: *mut i64) -> c_int;
    pub fn b200_net_set_tensor(net: *mut b200_net, name: *const c_char, kind: c_int, host: *const f32, n: i64) -> c_int;
    pub fn b200_net_get_tensor(net: *mut b200_net, name: *const c_char, kind: c_int, host: *mut f32, n: i64) -> c_int;
    pub fn b200_net_set_adamw(net: *mut b200_net, name: *const c_char, params: *const b200_adamw_params) -> c_int;

    pub fn b200_batch_upload(
        net: *mut b200_net,
        slot: c_int,
        stm: *const i32,
        nstm: *const i32,
        buckets: *const i32,
        targets: *const f32,
        n: i32,
    ) -> c_int;

    pub fn b200_batch_upload_records(
        net: *mut b200_net,
        slot: c_int,
        records: *const c_void,
        n: i32,
        game: i32,
        layout32: *const i32,
        scale: f32,
        blend: f32,
    ) -> c_int;

    pub fn b200_batch_upload_records_gpu(
        net: *mut b200_net,
        slot: c_int,
        records: *const c_void,
        n: i32,
        game: i32,
        layout32: *const i32,
        scale: f32,
        blend: f32,
    ) -> c_int;
    pub fn b200_slot_read(
        net: *mut b200_net,
        slot: c_int,
        stm: *mut u16,
        nstm: *mut u16,
        buckets: *mut i32,
        targets: *mut f32,
        order: *mut i32,
        pair_order: *mut i32,
        n: *mut i32,
    ) -> c_int;
    pub fn b200_net_set_optimiser(net: *mut b200_net, name: *const c_char, params: *const b200_optimiser_params) -> c_int;
    pub fn b200_probe_bandwidth(device: c_int, kind: c_int, bytes: i64, reps: c_int, gb_per_s: *mut f64) -> c_int;
    pub fn b200_step(net: *mut b200_net, slot: c_int, lr: f32, grad_factor: f32) -> c_int;
    pub fn b200_backward(net: *mut b200_net, slot: c_int) -> c_int;
    pub fn b200_update(net: *mut b200_net, lr: f32, grad_factor: f32) -> c_int;
    pub fn b200_grad_buffer(net: *mut b200_net, device_ptr: *mut *mut c_void, n_floats: *mut i64) -> c_int;
    pub fn b200_forward_begin(net: *mut b200_net, slot: c_int) -> c_int;
    pub fn b200_forward_ft(net: *mut b200_net, slot: c_int, part: c_int, n_parts: c_int) -> c_int;
    pub fn b200_net_tensor_offset(net: *mut b200_net, name: *const c_char, first_float: *mut i64) -> c_int;
    pub fn b200_exchange_export(net: *mut b200_net, handles: *mut c_void, bytes: i64) -> c_int;
    pub fn b200_exchange_import(net: *mut b200_net, rank: c_int, world: c_int, handles: *const c_void, bytes: i64) -> c_int;
    pub fn b200_update_exchange(net: *mut b200_net, lr: f32, grad_factor: f32) -> c_int;
    /// One data-parallel step with the exchange hidden under the feature-transformer backward.
    pub fn b200_step_exchange(net: *mut b200_net, slot: c_int, lr: f32, grad_factor: f32) -> c_int;
    pub fn b200_update_exchange_range(
        net: *mut b200_net,
        lr: f32,
        grad_factor: f32,
        first_float: i64,
        n_floats: i64,
        gather: c_int,
        stream: *mut c_void,
    ) -> c_int;
    pub fn b200_grad_zero_range(net: *mut b200_net, first_float: i64, n_floats: i64) -> c_int;
    pub fn b200_backward_begin(net: *mut b200_net, slot: c_int) -> c_int;
    pub fn b200_backward_ft(net: *mut b200_net, slot: c_int, part: c_int, n_parts: c_int) -> c_int;
    pub fn b200_backward_end(net: *mut b200_net, slot: c_int) -> c_int;
    pub fn b200_grad_part(net: *mut b200_net, part: c_int, n_parts: c_int, first_float: *mut i64, n_floats: *mut i64) -> c_int;
    pub fn b200_update_range(net: *mut b200_net, lr: f32, grad_factor: f32, first_float: i64, n_floats: i64) -> c_int;
    pub fn b200_update_end(net: *mut b200_net) -> c_int;
    pub fn b200_flat_buffer(net: *mut b200_net, kind: c_int, device_ptr: *mut *mut c_void, n_floats: *mut i64) -> c_int;
    pub fn b200_loss(net: *mut b200_net, loss_sum: *mut f32) -> c_int;
    pub fn b200_loss_of(net: *mut b200_net, steps_back: c_int, loss_sum: *mut f32) -> c_int;
    pub fn b200_forward(net: *mut b200_net, slot: c_int, out_host: *mut f32) -> c_int;
    pub fn b200_sync(net: *mut b200_net) -> c_int;
    pub fn b200_get_timings(net: *mut b200_net, out: *mut b200_timings) -> c_int;
    pub fn b200_net_get_stat(net: *mut b200_net, key: *const c_char, value: *mut i64) -> c_int;
    pub fn b200_net_get_activation(net: *mut b200_net, which: c_int, host: *mut f32, n: i64) -> c_int;

    pub fn b200_checkpoint_save(net: *mut b200_net, dir: *const c_char) -> c_int;
    pub fn b200_checkpoint_load(net: *mut b200_net, dir: *const c_char) -> c_int;

    pub fn b200_net_tensor_shape(net: *mut b200_net, name: *const c_char, rows: *mut i64, cols: *mut i64) -> c_int;
    pub fn b200_quant_size(quant: i32) -> i64;
    pub fn b200_quantise(values: *const f32, n: i64, quant: i32, multiplier: i32, round: i32, out: *mut c_void) -> c_int;
    pub fn b200_transpose(input: *const f32, rows: i64, cols: i64, out: *mut f32) -> c_int;
    pub fn b200_saved_format_size(net: *mut b200_net, fmt: *const b200_saved_format, n_fmt: i32, pad: i32, bytes: *mut i64) -> c_int;
    pub fn b200_saved_format_write(
        net: *mut b200_net,
        fmt: *const b200_saved_format,
        n_fmt: i32,
        pad: i32,
        out: *mut c_void,
        out_bytes: i64,
    ) -> c_int;
    pub fn b200_save_quantised(net: *mut b200_net, fmt: *const b200_saved_format, n_fmt: i32, path: *const c_char) -> c_int;
    pub fn b200_save_unquantised(net: *mut b200_net, fmt: *const b200_saved_format, n_fmt: i32, path: *const c_char) -> c_int;

    pub fn b200_op_ft_forward(device: c_int, stream: *mut c_void, op: *const b200_ft_op) -> c_int;
    pub fn b200_op_ft_forward_noalloc(device: c_int, stream: *mut c_void, op: *const b200_ft_op) -> c_int;

    pub fn b200_map_chess768(records: *const c_void, n: i32, stm: *mut i32, nstm: *mut i32, nnz: i32) -> c_int;
    pub fn b200_map_chess_buckets_mirrored(
        records: *const c_void,
        n: i32,
        layout32: *const i32,
        stm: *mut i32,
        nstm: *mut i32,
        nnz: i32,
    ) -> c_int;
    pub fn b200_map_ataxx147(records: *const c_void, n: i32, stm: *mut i32, nstm: *mut i32, nnz: i32) -> c_int;
    pub fn b200_material_count(records: *const c_void, n: i32, n_buckets: i32, out: *mut i32) -> c_int;
    pub fn b200_make_targets(records: *const c_void, n: i32, scale: f32, blend: f32, out: *mut f32) -> c_int;
    pub fn b200_set_host_threads(n: i32) -> c_int;
    pub fn b200_pack_indices_u16(idx: *const i32, count: i64, out: *mut u16) -> c_int;
    pub fn b200_unpack_indices_u16(packed: *const u16, count: i64, out: *mut i32) -> c_int;
}
