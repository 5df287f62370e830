//! Bindings of `libteeny_b200.so` (the sm_100a backend for the GEMM / flash-attention / Qwen3-forward path) for
//! `drivers/teeny-cuda`, and the direct-call launch path that stands where `CudaDevice::launch_with_packer`
//! (`drivers/teeny-cuda/src/device/mod.rs:430`) calls `cuLaunchKernel`.
//!
//! How it fits.  A lowered graph node is a `KernelExecutable { entry_point, kernel_source, runtime_op, .. }`
//! (`kernels/teeny-kernels/src/graph/mod.rs:2930-2951`).  The executor asks the node's `RuntimeOp` to `pack_args` into
//! an `ArgVisitor` and launches the compiled PTX.  The ops in `teeny-kernels/src/b200_ops.rs` have an empty
//! `kernel_source` and an `entry_point` that names a C function of this library; for those the executor hands the
//! visitor below (`B200ArgCollector`) to `pack_args` and calls `launch_direct(entry_point, &args, stream)` instead of
//! `cuLaunchKernel`.  The argument order a `RuntimeOp` packs is the C function's argument order; the launcher's two
//! trailing scratch pointers (`device/mod.rs:336-362`) become the `global_scratch` pair where a function has one, and
//! the stream comes last.
//!
//! The `extern "C"` block, the `#[repr(C)]` structs and the constants are generated from `include/teeny_b200.h` and
//! `include/teeny_qwen3.h` by `integration/cabi.py`; do not edit between the markers.
//!
//! `build.rs` of teeny-cuda gains: `println!("cargo:rustc-link-search=native={}", env!("TEENY_B200_LIB_DIR"));`

use core::ffi::{c_char, c_int, c_longlong, c_uint, c_ulonglong, c_void};
use std::ffi::CStr;

use teeny_core::device::program::ArgVisitor;

/// `cudaStream_t` / `CUstream`.
pub type CUstream = *mut c_void;

// ---- generated from include/*.h: begin ----
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct TeenyAttnShape {
    pub b: c_int,
    pub hq: c_int,
    pub hkv: c_int,
    pub sq: c_int,
    pub skv: c_int,
    pub d: c_int,
    pub q_sb: c_longlong,
    pub q_sh: c_longlong,
    pub q_ss: c_longlong,
    pub k_sb: c_longlong,
    pub k_sh: c_longlong,
    pub k_ss: c_longlong,
    pub v_sb: c_longlong,
    pub v_sh: c_longlong,
    pub v_ss: c_longlong,
    pub o_sb: c_longlong,
    pub o_sh: c_longlong,
    pub o_ss: c_longlong,
    pub scale: f32,
    pub causal: c_int,
}
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct TeenyQwen3Config {
    pub num_layers: c_int,
    pub hidden: c_int,
    pub num_q_heads: c_int,
    pub num_kv_heads: c_int,
    pub head_dim: c_int,
    pub intermediate: c_int,
    pub vocab: c_int,
    pub eps: f32,
    pub max_batch: c_int,
    pub max_len: c_int,
    pub max_tokens: c_int,
    pub max_new_tokens: c_int,
    pub tp_rank: c_int,
    pub tp_size: c_int,
}
/// Opaque runner handle (`teeny_qwen3`).
#[repr(C)]
pub struct TeenyQwen3 {
    _private: [u8; 0],
}
pub const TEENY_OK: c_int = 0;
pub const TEENY_ERR_BAD_ARG: c_int = -1;
pub const TEENY_ERR_ALIGNMENT: c_int = -2;
pub const TEENY_ERR_SCRATCH: c_int = -3;
pub const TEENY_ERR_DRIVER: c_int = -4;
pub const TEENY_ERR_DEVICE_WAIT: c_int = -5;
pub const TEENY_ERR_NCCL: c_int = -6;
pub const TEENY_ERR_STATIC_LIMIT: c_int = -7;
pub const TEENY_QWEN3_W_QKV: c_int = 0;
pub const TEENY_QWEN3_W_O: c_int = 1;
pub const TEENY_QWEN3_W_GATE_UP: c_int = 2;
pub const TEENY_QWEN3_W_DOWN: c_int = 3;
pub const TEENY_QWEN3_W_INPUT_LN: c_int = 4;
pub const TEENY_QWEN3_W_POST_LN: c_int = 5;
pub const TEENY_QWEN3_W_Q_NORM: c_int = 6;
pub const TEENY_QWEN3_W_K_NORM: c_int = 7;
pub const TEENY_QWEN3_W_EMBED: c_int = 100;
pub const TEENY_QWEN3_W_FINAL_NORM: c_int = 101;
pub const TEENY_QWEN3_W_LM_HEAD: c_int = 102;
pub const TEENY_QWEN3_W_INV_FREQ: c_int = 103;
pub const TEENY_QWEN3_BUF_LOGITS: c_int = 0;
pub const TEENY_QWEN3_BUF_NEXT_IDS: c_int = 1;
pub const TEENY_QWEN3_BUF_HISTORY: c_int = 2;
pub const TEENY_QWEN3_BUF_STATE: c_int = 3;
pub const TEENY_QWEN3_BUF_HIDDEN: c_int = 4;
pub const TEENY_QWEN3_BUF_K_CACHE: c_int = 5;
pub const TEENY_QWEN3_BUF_V_CACHE: c_int = 6;
pub const TEENY_QWEN3_BUF_RESIDUAL: c_int = 7;
pub const TEENY_QWEN3_BUF_LAST_DELTA: c_int = 8;
#[link(name = "teeny_b200")]
extern "C" {
    pub fn teeny_version() -> c_int;
    pub fn teeny_status_string(status: c_int) -> *const c_char;
    pub fn teeny_device_error(clear: c_int) -> c_int;
    pub fn teeny_launch_count(reset: c_int) -> c_ulonglong;
    pub fn matmul_forward_entry_point_f32(a: *const f32, b: *const f32, c: *mut f32, m: c_int, n: c_int, k: c_int, global_scratch: *mut c_void, global_scratch_bytes: usize, stream: CUstream) -> c_int;
    pub fn matmul_forward_entry_point_bf16(a: *const u16, b: *const u16, c: *mut u16, m: c_int, n: c_int, k: c_int, global_scratch: *mut c_void, global_scratch_bytes: usize, stream: CUstream) -> c_int;
    pub fn linear_forward_entry_point_f32(x: *const f32, w: *const f32, bias: *const f32, y: *mut f32, m: c_int, n: c_int, k: c_int, stride_xm: c_int, stride_xk: c_int, stride_wn: c_int, stride_wk: c_int, stride_ym: c_int, stride_yn: c_int, global_scratch: *mut c_void, global_scratch_bytes: usize, stream: CUstream) -> c_int;
    pub fn linear_forward_entry_point_bf16(x: *const u16, w: *const u16, bias: *const u16, y: *mut u16, m: c_int, n: c_int, k: c_int, stride_xm: c_int, stride_xk: c_int, stride_wn: c_int, stride_wk: c_int, stride_ym: c_int, stride_yn: c_int, global_scratch: *mut c_void, global_scratch_bytes: usize, stream: CUstream) -> c_int;
    pub fn teeny_matmul_f32_scratch_bytes(m: c_int, n: c_int, k: c_int) -> usize;
    pub fn teeny_gemm_scratch_bytes(m: c_int, n: c_int, k: c_int) -> usize;
    pub fn flash_attention2_forward_entry_point_f32(q: *const f32, k: *const f32, v: *const f32, o: *mut f32, l: *mut f32, n_ctx_q: c_int, n_ctx_k: c_int, softmax_scale: f32, neg_inf: f32, bh: c_int, head_dim: c_int, stream: CUstream) -> c_int;
    pub fn flash_attention2_forward_entry_point_bf16(q: *const u16, k: *const u16, v: *const u16, o: *mut u16, l: *mut f32, n_ctx_q: c_int, n_ctx_k: c_int, softmax_scale: f32, neg_inf: f32, bh: c_int, head_dim: c_int, stream: CUstream) -> c_int;
    pub fn teeny_flash_attn_fwd_bf16(q: *const u16, k: *const u16, v: *const u16, o: *mut u16, lse: *mut f32, shape: *const TeenyAttnShape, stream: CUstream) -> c_int;
    pub fn teeny_flash_attn_decode_bf16(q: *const u16, k: *const u16, v: *const u16, o: *mut u16, shape: *const TeenyAttnShape, kv_len: c_int, kv_len_dev: *const c_int, scratch: *mut c_void, scratch_bytes: usize, stream: CUstream) -> c_int;
    pub fn teeny_attn_decode_scratch_bytes(b: c_int, hq: c_int, d: c_int, max_kv: c_int) -> usize;
    pub fn teeny_flash_attn_decode_bf16_static(q: *const u16, k: *const u16, v: *const u16, o: *mut u16, shape: *const TeenyAttnShape, kv_len: c_int, kv_len_dev: *const c_int, stream: CUstream) -> c_int;
    pub fn teeny_attn_decode_static_limit() -> usize;
    pub fn rms_norm_forward_entry_point_f32(x: *const f32, y: *mut f32, weight: *const f32, rrms: *mut f32, m: c_int, n: c_int, eps: f32, stream: CUstream) -> c_int;
    pub fn rms_norm_forward_entry_point_bf16(x: *const u16, y: *mut u16, weight: *const u16, rrms: *mut f32, m: c_int, n: c_int, eps: f32, stream: CUstream) -> c_int;
    pub fn silu_forward_entry_point_f32(x: *const f32, y: *mut f32, n: c_int, stream: CUstream) -> c_int;
    pub fn silu_forward_entry_point_bf16(x: *const u16, y: *mut u16, n: c_int, stream: CUstream) -> c_int;
    pub fn elemwise_mul_forward_entry_point_f32(a: *const f32, b: *const f32, out: *mut f32, n: c_int, stream: CUstream) -> c_int;
    pub fn elemwise_mul_forward_entry_point_bf16(a: *const u16, b: *const u16, out: *mut u16, n: c_int, stream: CUstream) -> c_int;
    pub fn elemwise_add_forward_entry_point_f32(a: *const f32, b: *const f32, out: *mut f32, n: c_int, stream: CUstream) -> c_int;
    pub fn elemwise_add_forward_entry_point_bf16(a: *const u16, b: *const u16, out: *mut u16, n: c_int, stream: CUstream) -> c_int;
    pub fn softmax_forward_entry_point_f32(x: *const f32, y: *mut f32, n_rows: c_int, n_cols: c_int, stream: CUstream) -> c_int;
    pub fn softmax_forward_entry_point_bf16(x: *const u16, y: *mut u16, n_rows: c_int, n_cols: c_int, stream: CUstream) -> c_int;
    pub fn teeny_add_rms_norm_bf16(x: *const u16, residual: *mut u16, y: *mut u16, weight: *const u16, m: c_int, n: c_int, eps: f32, stream: CUstream) -> c_int;
    pub fn teeny_silu_mul_bf16(gate_up: *const u16, ld: c_longlong, out: *mut u16, t: c_int, inter: c_int, stream: CUstream) -> c_int;
    pub fn teeny_linear_swiglu_bf16(x: *const u16, ldx: c_longlong, w: *const u16, ldw: c_longlong, y: *mut u16, ldy: c_longlong, m: c_int, n: c_int, k: c_int, stream: CUstream) -> c_int;
    pub fn teeny_linear_w8a16_forward(x: *const u16, ldx: c_longlong, w_fp8: *const c_void, ldw: c_longlong, w_scale: *const f32, scale_kind: c_int, group_size: c_int, bias: *const u16, y: *mut u16, ldy: c_longlong, m: c_int, n: c_int, k: c_int, swiglu: c_int, global_scratch: *mut c_void, global_scratch_bytes: usize, stream: CUstream) -> c_int;
    pub fn teeny_linear_w8a16_scratch_bytes(m: c_int, n: c_int, k: c_int) -> usize;
    pub fn teeny_split_fp8_e4m3(x: *const u16, ldx: c_longlong, out: *mut c_void, ldo: c_longlong, x_scale: *mut f32, m: c_int, k: c_int, stream: CUstream) -> c_int;
    pub fn teeny_linear_w8a8x2_forward(x_fp8: *const c_void, ldx: c_longlong, x_scale: *const f32, w_fp8: *const c_void, ldw: c_longlong, w_scale: *const f32, scale_kind: c_int, bias: *const u16, y: *mut u16, ldy: c_longlong, m: c_int, n: c_int, k: c_int, swiglu: c_int, stream: CUstream) -> c_int;
    pub fn teeny_dequant_fp8_e4m3_bf16(w_fp8: *const c_void, ldw: c_longlong, w_scale: *const f32, scale_kind: c_int, group_size: c_int, out: *mut u16, ldo: c_longlong, n: c_int, k: c_int, stream: CUstream) -> c_int;
    pub fn teeny_dequant_int_bf16(q: *const c_void, bits: c_int, w_scale: *const f32, zero_point: *const c_int, scale_kind: c_int, group_size: c_int, out: *mut u16, ldo: c_longlong, n: c_int, k: c_int, stream: CUstream) -> c_int;
    pub fn teeny_fp8_e4m3_count_nan(bytes: *const c_void, n: usize, count: *mut c_uint, stream: CUstream) -> c_int;
    pub fn teeny_rope_table_bf16(inv_freq: *const f32, cos_table: *mut u16, sin_table: *mut u16, max_pos: c_int, d: c_int, stream: CUstream) -> c_int;
    pub fn teeny_qk_norm_rope_kv_bf16(qkv: *mut u16, ld: c_longlong, q_norm_w: *const u16, k_norm_w: *const u16, cos_table: *const u16, sin_table: *const u16, k_cache: *mut u16, v_cache: *mut u16, t: c_int, s: c_int, hq: c_int, hkv: c_int, d: c_int, max_len: c_int, pos0: c_int, pos0_dev: *const c_int, eps: f32, stream: CUstream) -> c_int;
    pub fn teeny_embedding_bf16(ids: *const c_int, table: *const u16, out: *mut u16, t: c_int, hidden: c_int, vocab: c_int, stream: CUstream) -> c_int;
    pub fn teeny_argmax_bf16(logits: *const u16, ld: c_longlong, best_val: *mut f32, best_idx: *mut c_int, rows: c_int, cols: c_int, idx_offset: c_int, stream: CUstream) -> c_int;
    pub fn teeny_argmax_combine(vals: *const f32, idx: *const c_int, out_idx: *mut c_int, parts: c_int, rows: c_int, stream: CUstream) -> c_int;
    pub fn teeny_sample_top_k_top_p_bf16(logits: *const u16, ld: c_longlong, rows: c_int, cols: c_int, temperature: f32, top_k: c_int, top_p: f32, u: *const f32, out_idx: *mut c_int, out_prob: *mut f32, stream: CUstream) -> c_int;
    pub fn teeny_sample_candidates_bf16(logits: *const u16, ld: c_longlong, rows: c_int, cols: c_int, top_k: c_int, idx_offset: c_int, cand_out: *mut c_ulonglong, stream: CUstream) -> c_int;
    pub fn teeny_sample_merge(lists: *const c_ulonglong, parts: c_int, list_stride: usize, rows: c_int, temperature: f32, top_k: c_int, top_p: f32, u: *const f32, out_idx: *mut c_int, out_prob: *mut f32, stream: CUstream) -> c_int;
    pub fn teeny_qwen3_workspace_bytes(cfg: *const TeenyQwen3Config) -> usize;
    pub fn teeny_qwen3_create(cfg: *const TeenyQwen3Config, workspace: *mut c_void, workspace_bytes: usize, tp_comm: *mut c_void, stream: CUstream, out: *mut *mut TeenyQwen3) -> c_int;
    pub fn teeny_qwen3_destroy(model: *mut TeenyQwen3);
    pub fn teeny_qwen3_set_weight(model: *mut TeenyQwen3, layer: c_int, which: c_int, device_ptr: *const c_void) -> c_int;
    pub fn teeny_qwen3_set_weight_fp8(model: *mut TeenyQwen3, layer: c_int, which: c_int, fp8_bytes: *const c_void, scales: *const f32, scale_kind: c_int, group_size: c_int) -> c_int;
    pub fn teeny_qwen3_fp8_scratch_bytes(cfg: *const TeenyQwen3Config) -> usize;
    pub fn teeny_qwen3_set_fp8_scratch(model: *mut TeenyQwen3, scratch: *mut c_void, bytes: usize) -> c_int;
    pub fn teeny_qwen3_prefill(model: *mut TeenyQwen3, ids: *const c_int, b: c_int, s: c_int, stream: CUstream) -> c_int;
    pub fn teeny_qwen3_decode(model: *mut TeenyQwen3, stream: CUstream) -> c_int;
    pub fn teeny_qwen3_set_sampling(model: *mut TeenyQwen3, temperature: f32, top_k: c_int, top_p: f32, seed: c_ulonglong) -> c_int;
    pub fn teeny_qwen3_capture_decode(model: *mut TeenyQwen3, stream: CUstream) -> c_int;
    pub fn teeny_qwen3_decode_replay(model: *mut TeenyQwen3, stream: CUstream) -> c_int;
    pub fn teeny_qwen3_buffer(model: *mut TeenyQwen3, which: c_int) -> *mut c_void;
    pub fn teeny_tp_unique_id(out128: *mut c_void) -> c_int;
    pub fn teeny_tp_init(id128: *const c_void, rank: c_int, world: c_int, comm_out: *mut *mut c_void) -> c_int;
    pub fn teeny_tp_destroy(comm: *mut c_void) -> c_int;
    pub fn teeny_tp_all_reduce_bf16(comm: *mut c_void, buf: *mut u16, count: usize, stream: CUstream) -> c_int;
    pub fn teeny_tp_peer_enabled(comm: *mut c_void) -> c_int;
    pub fn teeny_tp_gather_add_rms_norm_bf16(recv: *const c_void, slot_elems: usize, world: c_int, epoch: *const u32, round: u32, residual: *mut u16, y: *mut u16, weight: *const u16, m: c_int, n: c_int, eps: f32, wait_limit_ns: c_ulonglong, stream: CUstream) -> c_int;
}
// ---- generated from include/*.h: end ----

/// One packed kernel argument, as a `RuntimeOp` hands it to an `ArgVisitor`.
#[derive(Clone, Copy, Debug, PartialEq)]
pub enum Arg {
    Ptr(*mut c_void),
    I32(i32),
    I64(i64),
    F32(f32),
}

/// The `ArgVisitor` of the direct-call path: keeps the arguments typed instead of flattening them into the byte
/// buffers `CudaArgPacker` builds for `cuLaunchKernel` (`device/mod.rs:49-113`).
#[derive(Default)]
pub struct B200ArgCollector {
    pub args: Vec<Arg>,
}

impl ArgVisitor for B200ArgCollector {
    fn visit_ptr(&mut self, ptr: *mut c_void) {
        self.args.push(Arg::Ptr(ptr));
    }
    fn visit_bool(&mut self, val: bool) {
        self.args.push(Arg::I32(val as i32));
    }
    fn visit_i8(&mut self, val: i8) {
        self.args.push(Arg::I32(val as i32));
    }
    fn visit_i16(&mut self, val: i16) {
        self.args.push(Arg::I32(val as i32));
    }
    fn visit_i32(&mut self, val: i32) {
        self.args.push(Arg::I32(val));
    }
    fn visit_i64(&mut self, val: i64) {
        self.args.push(Arg::I64(val));
    }
    fn visit_u8(&mut self, val: u8) {
        self.args.push(Arg::I32(val as i32));
    }
    fn visit_u16(&mut self, val: u16) {
        self.args.push(Arg::I32(val as i32));
    }
    fn visit_u32(&mut self, val: u32) {
        self.args.push(Arg::I64(val as i64));
    }
    fn visit_u64(&mut self, val: u64) {
        self.args.push(Arg::I64(val as i64));
    }
    fn visit_f32(&mut self, val: f32) {
        self.args.push(Arg::F32(val));
    }
    fn visit_f64(&mut self, val: f64) {
        self.args.push(Arg::F32(val as f32));
    }
}

/// Maps a status of this library onto the crate's error type (0 ok, negative = rejected call, positive = cudaError_t).
pub fn check(status: c_int, what: &str) -> anyhow::Result<()> {
    if status == 0 {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(teeny_status_string(status)) }.to_string_lossy().into_owned();
    Err(anyhow::anyhow!("teeny_b200: {what}: status {status} ({msg})"))
}

fn p(a: &[Arg], i: usize) -> *mut c_void {
    match a[i] {
        Arg::Ptr(v) => v,
        other => panic!("argument {i}: expected a pointer, got {other:?}"),
    }
}
fn i(a: &[Arg], k: usize) -> c_int {
    match a[k] {
        Arg::I32(v) => v,
        other => panic!("argument {k}: expected an i32, got {other:?}"),
    }
}
fn l(a: &[Arg], k: usize) -> c_longlong {
    match a[k] {
        Arg::I64(v) => v,
        Arg::I32(v) => v as c_longlong,
        other => panic!("argument {k}: expected an i64, got {other:?}"),
    }
}
fn f(a: &[Arg], k: usize) -> f32 {
    match a[k] {
        Arg::F32(v) => v,
        other => panic!("argument {k}: expected an f32, got {other:?}"),
    }
}

/// Calls the library function named `entry_point` with the arguments a `RuntimeOp` packed, on `stream`.
/// Launches do not synchronise (the reference calls `cuCtxSynchronize` after every launch, `device/mod.rs:369-381`):
/// call `device_error()` where that behaviour is wanted.
pub fn launch_direct(entry_point: &str, a: &[Arg], stream: CUstream) -> anyhow::Result<()> {
    let null = core::ptr::null_mut::<c_void>();
    let st = unsafe {
        match entry_point {
            "matmul_forward_entry_point_f32" => matmul_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), i(a, 4), i(a, 5), null, 0, stream),
            "matmul_forward_entry_point_bf16" => matmul_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), i(a, 4), i(a, 5), null, 0, stream),
            "linear_forward_entry_point_f32" => linear_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), p(a, 3).cast(), i(a, 4), i(a, 5), i(a, 6), i(a, 7), i(a, 8), i(a, 9), i(a, 10), i(a, 11), i(a, 12), null, 0, stream),
            "linear_forward_entry_point_bf16" => linear_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), p(a, 3).cast(), i(a, 4), i(a, 5), i(a, 6), i(a, 7), i(a, 8), i(a, 9), i(a, 10), i(a, 11), i(a, 12), null, 0, stream),
            "rms_norm_forward_entry_point_f32" => rms_norm_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), p(a, 3).cast(), i(a, 4), i(a, 5), f(a, 6), stream),
            "rms_norm_forward_entry_point_bf16" => rms_norm_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), p(a, 3).cast(), i(a, 4), i(a, 5), f(a, 6), stream),
            "silu_forward_entry_point_f32" => silu_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), i(a, 2), stream),
            "silu_forward_entry_point_bf16" => silu_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), i(a, 2), stream),
            "elemwise_mul_forward_entry_point_f32" => elemwise_mul_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), stream),
            "elemwise_mul_forward_entry_point_bf16" => elemwise_mul_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), stream),
            "elemwise_add_forward_entry_point_f32" => elemwise_add_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), stream),
            "elemwise_add_forward_entry_point_bf16" => elemwise_add_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), stream),
            "softmax_forward_entry_point_f32" => softmax_forward_entry_point_f32(p(a, 0).cast(), p(a, 1).cast(), i(a, 2), i(a, 3), stream),
            "softmax_forward_entry_point_bf16" => softmax_forward_entry_point_bf16(p(a, 0).cast(), p(a, 1).cast(), i(a, 2), i(a, 3), stream),
            "teeny_add_rms_norm_bf16" => teeny_add_rms_norm_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), p(a, 3).cast(), i(a, 4), i(a, 5), f(a, 6), stream),
            "teeny_silu_mul_bf16" => teeny_silu_mul_bf16(p(a, 0).cast(), l(a, 1), p(a, 2).cast(), i(a, 3), i(a, 4), stream),
            "teeny_linear_swiglu_bf16" => teeny_linear_swiglu_bf16(p(a, 0).cast(), l(a, 1), p(a, 2).cast(), l(a, 3), p(a, 4).cast(), l(a, 5), i(a, 6), i(a, 7), i(a, 8), stream),
            "teeny_qk_norm_rope_kv_bf16" => teeny_qk_norm_rope_kv_bf16(p(a, 0).cast(), l(a, 1), p(a, 2).cast(), p(a, 3).cast(), p(a, 4).cast(), p(a, 5).cast(), p(a, 6).cast(), p(a, 7).cast(), i(a, 8), i(a, 9), i(a, 10), i(a, 11), i(a, 12), i(a, 13), i(a, 14), p(a, 15).cast(), f(a, 16), stream),
            "teeny_flash_attn_fwd_bf16" => teeny_flash_attn_fwd_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), p(a, 3).cast(), p(a, 4).cast(), p(a, 5).cast(), stream),
            "teeny_embedding_bf16" => teeny_embedding_bf16(p(a, 0).cast(), p(a, 1).cast(), p(a, 2).cast(), i(a, 3), i(a, 4), i(a, 5), stream),
            "teeny_argmax_bf16" => teeny_argmax_bf16(p(a, 0).cast(), l(a, 1), p(a, 2).cast(), p(a, 3).cast(), i(a, 4), i(a, 5), i(a, 6), stream),
            other => return Err(anyhow::anyhow!("teeny_b200: no direct-call binding for entry point '{other}'")),
        }
    };
    check(st, entry_point)
}

/// Synchronises the device and returns the error word the kernels set when one of their bounded waits expires.
pub fn device_error(clear: bool) -> anyhow::Result<()> {
    match unsafe { teeny_device_error(clear as c_int) } {
        0 => Ok(()),
        word if word > 0 && word < 0x1000 => Err(anyhow::anyhow!("teeny_b200: a kernel gave up on a bounded wait (role {word:#x})")),
        other => check(other, "teeny_device_error"),
    }
}

/// Qwen3 decoder runner: `LoadedModel::forward` / `capture_graph` / `CudaGraphModel::run`
/// (`drivers/teeny-cuda/src/model/mod.rs:524, 1245, 1799`) for the one graph this backend executes end to end.
/// The caller owns the workspace and the weights (device memory); this type owns only the small host-side handle.
pub struct Qwen3Runner {
    handle: *mut TeenyQwen3,
    stream: CUstream,
}

// the handle is only touched through &mut self
unsafe impl Send for Qwen3Runner {}

impl Qwen3Runner {
    pub fn workspace_bytes(cfg: &TeenyQwen3Config) -> usize {
        unsafe { teeny_qwen3_workspace_bytes(cfg) }
    }

    /// `workspace`: device memory of at least `workspace_bytes(cfg)` bytes, 256-byte aligned.
    pub fn new(cfg: &TeenyQwen3Config, workspace: *mut c_void, workspace_bytes: usize, tp_comm: *mut c_void, stream: CUstream) -> anyhow::Result<Self> {
        let mut handle = core::ptr::null_mut();
        check(unsafe { teeny_qwen3_create(cfg, workspace, workspace_bytes, tp_comm, stream, &mut handle) }, "teeny_qwen3_create")?;
        Ok(Self { handle, stream })
    }

    /// `which`: one of the `TEENY_QWEN3_W_*` slots; `layer` is ignored for the model-level ones.
    pub fn set_weight(&mut self, layer: i32, which: c_int, device_ptr: *const c_void) -> anyhow::Result<()> {
        check(unsafe { teeny_qwen3_set_weight(self.handle, layer, which, device_ptr) }, "teeny_qwen3_set_weight")
    }

    pub fn prefill(&mut self, ids: *const c_int, batch: i32, prompt_len: i32) -> anyhow::Result<()> {
        check(unsafe { teeny_qwen3_prefill(self.handle, ids, batch, prompt_len, self.stream) }, "teeny_qwen3_prefill")
    }

    pub fn decode(&mut self) -> anyhow::Result<()> {
        check(unsafe { teeny_qwen3_decode(self.handle, self.stream) }, "teeny_qwen3_decode")
    }

    pub fn capture_decode(&mut self) -> anyhow::Result<()> {
        check(unsafe { teeny_qwen3_capture_decode(self.handle, self.stream) }, "teeny_qwen3_capture_decode")
    }

    pub fn decode_replay(&mut self) -> anyhow::Result<()> {
        check(unsafe { teeny_qwen3_decode_replay(self.handle, self.stream) }, "teeny_qwen3_decode_replay")
    }

    pub fn set_sampling(&mut self, temperature: f32, top_k: i32, top_p: f32, seed: u64) -> anyhow::Result<()> {
        check(unsafe { teeny_qwen3_set_sampling(self.handle, temperature, top_k, top_p, seed as c_ulonglong) }, "teeny_qwen3_set_sampling")
    }

    /// Device address of one of the runner's buffers (`TEENY_QWEN3_BUF_*`).
    pub fn buffer(&self, which: c_int) -> *mut c_void {
        unsafe { teeny_qwen3_buffer(self.handle, which) }
    }
}

impl Drop for Qwen3Runner {
    fn drop(&mut self) {
        unsafe { teeny_qwen3_destroy(self.handle) }
    }
}
