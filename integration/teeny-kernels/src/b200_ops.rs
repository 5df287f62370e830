//! Graph ops that lower onto `libteeny_b200.so` through the sanctioned plug-in hook `CustomOp::lower()`
//! (`core/teeny-core/src/graph/mod.rs:109-133`, consumed at `kernels/teeny-kernels/src/graph/mod.rs:2930-2951`).
//!
//! Each op returns `(name, kernel_source = "", entry_point, runtime_op)`: the empty source tells the CUDA executor
//! that the entry point is a C function of the library (`drivers/teeny-cuda/src/b200.rs::launch_direct`), not a PTX
//! symbol.  `pack_args` visits the C function's arguments in declaration order, up to (not including) the scratch
//! pair and the stream, which the executor appends -- the same contract `RuntimeOp for LinearForward` follows for
//! its PTX kernel (`kernels/teeny-kernels/src/nn/mlp/linear.rs:275-307`).  `grid` / `block` are unused by the
//! direct-call path (the library sizes its own launches) and return one CTA of one warp.
//!
//! Ops:
//!   * `LinearB200`        `Op::Linear` (`graph/mod.rs:1105`) for bf16 activations: `linear_forward_entry_point_bf16`.
//!   * `RmsNormResidual`   residual add + RMSNorm, the pair `Op::Add` + `Op::RmsNorm` of every decoder block:
//!                         `teeny_add_rms_norm_bf16`.
//!   * `SwiGluMlp`         gate and up projections + SiLU + multiply in one GEMM: `teeny_linear_swiglu_bf16`.
//!   * `QwenAttention`     per-head q/k RMSNorm, rotary embedding, KV-cache fill and causal grouped-query attention:
//!                         `Op::RotaryEmbedding` and `Op::MultiHeadAttention`, which return `Err("TODO")` today
//!                         (`graph/mod.rs:2598-2607`); two launches, `teeny_qk_norm_rope_kv_bf16` then
//!                         `teeny_flash_attn_fwd_bf16`.

use std::any::Any;
use std::sync::{Arc, Mutex};

use teeny_core::device::program::ArgVisitor;
use teeny_core::graph::{CustomOp, Shape};
use teeny_core::model::{RawPtr, RuntimeOp};
use teeny_cuda::b200::TeenyAttnShape;

const ONE_WARP: [u32; 3] = [32, 1, 1];
const ONE_CTA: [u32; 3] = [1, 1, 1];

fn lowered(name: &str, entry_point: &str, op: Arc<dyn RuntimeOp>) -> Option<(String, String, String, Arc<dyn RuntimeOp>)> {
    Some((name.to_string(), String::new(), entry_point.to_string(), op))
}

// ---------------------------------------------------------------------------------------------------------------
// Linear: y[M, N] = x[M, K] w[N, K]^T (+ bias)
// ---------------------------------------------------------------------------------------------------------------
#[derive(Clone, Debug)]
pub struct LinearB200 {
    pub out_features: usize,
    pub use_bias: bool,
}

impl RuntimeOp for LinearB200 {
    fn n_activation_inputs(&self) -> usize {
        1
    }

    fn param_shapes(&self, input_shapes: &[&[usize]], output_shape: &[usize]) -> Vec<Vec<usize>> {
        let (k, n) = (input_shapes[0][1], output_shape[1]);
        if self.use_bias { vec![vec![n, k], vec![n]] } else { vec![vec![n, k]] }
    }

    fn param_names(&self) -> &'static [&'static str] {
        &["weight", "bias"]
    }

    // entry point: linear_forward_entry_point_bf16
    fn pack_args(&self, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], output: RawPtr, output_shape: &[usize],
                 output_row_stride: i32, visitor: &mut dyn ArgVisitor) {
        let (m, n, k) = (output_shape[0] as i32, output_shape[1] as i32, inputs[0].1[1] as i32);
        let bias = if self.use_bias { params[1] } else { core::ptr::null_mut() };
        visitor.visit_ptr(inputs[0].0); // x
        visitor.visit_ptr(params[0]); // w
        visitor.visit_ptr(bias); // bias
        visitor.visit_ptr(output); // y
        visitor.visit_i32(m); // M
        visitor.visit_i32(n); // N
        visitor.visit_i32(k); // K
        visitor.visit_i32(k); // stride_xm
        visitor.visit_i32(1); // stride_xk
        visitor.visit_i32(k); // stride_wn
        visitor.visit_i32(1); // stride_wk
        visitor.visit_i32(output_row_stride); // stride_ym
        visitor.visit_i32(1); // stride_yn
    }

    fn block(&self) -> [u32; 3] {
        ONE_WARP
    }

    fn grid(&self, _output_shape: &[usize]) -> [u32; 3] {
        ONE_CTA
    }
}

impl CustomOp for LinearB200 {
    fn name(&self) -> &str {
        "linear_b200"
    }

    fn infer_output_shape(&self, input_shapes: &[&Shape]) -> Shape {
        vec![input_shapes[0][0], Some(self.out_features)]
    }

    fn as_any(&self) -> &dyn Any {
        self
    }

    fn lower(&self) -> Option<(String, String, String, Arc<dyn RuntimeOp>)> {
        lowered("linear_b200", "linear_forward_entry_point_bf16", Arc::new(self.clone()))
    }
}

// ---------------------------------------------------------------------------------------------------------------
// RmsNormResidual: residual <- residual + x (in place); y = rms_norm(residual) * weight
// ---------------------------------------------------------------------------------------------------------------
#[derive(Clone, Debug)]
pub struct RmsNormResidual {
    pub eps: f32,
}

impl RuntimeOp for RmsNormResidual {
    fn n_activation_inputs(&self) -> usize {
        2 // x (the block's projection output), residual (updated in place)
    }

    fn param_shapes(&self, _input_shapes: &[&[usize]], output_shape: &[usize]) -> Vec<Vec<usize>> {
        vec![vec![output_shape[1]]]
    }

    fn param_names(&self) -> &'static [&'static str] {
        &["weight"]
    }

    // entry point: teeny_add_rms_norm_bf16
    fn pack_args(&self, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], output: RawPtr, output_shape: &[usize],
                 _output_row_stride: i32, visitor: &mut dyn ArgVisitor) {
        visitor.visit_ptr(inputs[0].0); // x
        visitor.visit_ptr(inputs[1].0); // residual
        visitor.visit_ptr(output); // y
        visitor.visit_ptr(params[0]); // weight
        visitor.visit_i32(output_shape[0] as i32); // M
        visitor.visit_i32(output_shape[1] as i32); // N
        visitor.visit_f32(self.eps); // eps
    }

    fn block(&self) -> [u32; 3] {
        ONE_WARP
    }

    fn grid(&self, _output_shape: &[usize]) -> [u32; 3] {
        ONE_CTA
    }
}

impl CustomOp for RmsNormResidual {
    fn name(&self) -> &str {
        "rms_norm_residual"
    }

    fn infer_output_shape(&self, input_shapes: &[&Shape]) -> Shape {
        input_shapes[1].clone()
    }

    fn as_any(&self) -> &dyn Any {
        self
    }

    fn lower(&self) -> Option<(String, String, String, Arc<dyn RuntimeOp>)> {
        lowered("rms_norm_residual", "teeny_add_rms_norm_bf16", Arc::new(self.clone()))
    }
}

// ---------------------------------------------------------------------------------------------------------------
// SwiGluMlp: y[M, I] = silu(x Wg^T) * (x Wu^T), one GEMM over the interleaved [2 I, K] gate / up weight
// ---------------------------------------------------------------------------------------------------------------
#[derive(Clone, Debug)]
pub struct SwiGluMlp {
    pub intermediate: usize,
}

impl SwiGluMlp {
    /// The `[2 I, K]` parameter this op expects: gate and up rows interleaved in blocks of 64 channels (rows
    /// `128 b .. 128 b + 63` = gate channels `64 b ..`, rows `128 b + 64 .. 128 b + 127` = up channels `64 b ..`), so a
    /// weight tile of the GEMM holds both projections of 64 channels and the epilogue applies SiLU and the product.
    pub fn interleave_gate_up<T: Copy>(gate: &[T], up: &[T], intermediate: usize, k: usize) -> Vec<T> {
        assert!(intermediate % 64 == 0 && gate.len() == intermediate * k && up.len() == intermediate * k);
        let mut out = Vec::with_capacity(2 * intermediate * k);
        for b in 0..intermediate / 64 {
            out.extend_from_slice(&gate[b * 64 * k..(b + 1) * 64 * k]);
            out.extend_from_slice(&up[b * 64 * k..(b + 1) * 64 * k]);
        }
        out
    }
}

impl RuntimeOp for SwiGluMlp {
    fn n_activation_inputs(&self) -> usize {
        1
    }

    fn param_shapes(&self, input_shapes: &[&[usize]], _output_shape: &[usize]) -> Vec<Vec<usize>> {
        vec![vec![2 * self.intermediate, input_shapes[0][1]]]
    }

    fn param_names(&self) -> &'static [&'static str] {
        &["gate_up_weight"]
    }

    // entry point: teeny_linear_swiglu_bf16
    fn pack_args(&self, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], output: RawPtr, output_shape: &[usize],
                 output_row_stride: i32, visitor: &mut dyn ArgVisitor) {
        let (m, k) = (output_shape[0] as i32, inputs[0].1[1] as i32);
        visitor.visit_ptr(inputs[0].0); // x
        visitor.visit_i64(k as i64); // ldx
        visitor.visit_ptr(params[0]); // w
        visitor.visit_i64(k as i64); // ldw
        visitor.visit_ptr(output); // y
        visitor.visit_i64(output_row_stride as i64); // ldy
        visitor.visit_i32(m); // M
        visitor.visit_i32(2 * self.intermediate as i32); // N
        visitor.visit_i32(k); // K
    }

    fn block(&self) -> [u32; 3] {
        ONE_WARP
    }

    fn grid(&self, _output_shape: &[usize]) -> [u32; 3] {
        ONE_CTA
    }
}

impl CustomOp for SwiGluMlp {
    fn name(&self) -> &str {
        "swiglu_mlp"
    }

    fn infer_output_shape(&self, input_shapes: &[&Shape]) -> Shape {
        vec![input_shapes[0][0], Some(self.intermediate)]
    }

    fn as_any(&self) -> &dyn Any {
        self
    }

    fn lower(&self) -> Option<(String, String, String, Arc<dyn RuntimeOp>)> {
        lowered("swiglu_mlp", "teeny_linear_swiglu_bf16", Arc::new(self.clone()))
    }
}

// ---------------------------------------------------------------------------------------------------------------
// QwenAttention: qkv[T, (Hq + 2 Hkv) 128] -> attn[T, Hq 128]
//   launch 0: per-head RMSNorm of q and k, rotary embedding, KV-cache fill   (teeny_qk_norm_rope_kv_bf16)
//   launch 1: causal grouped-query flash attention over the cache            (teeny_flash_attn_fwd_bf16)
// Parameters: q_norm.weight [128], k_norm.weight [128], rope cos / sin tables [max_len, 128] (bf16, built once with
// teeny_rope_table_bf16 from the model's inv_freq), k / v caches [B, Hkv, max_len, 128].
// ---------------------------------------------------------------------------------------------------------------
#[derive(Debug)]
pub struct QwenAttention {
    pub num_q_heads: usize,
    pub num_kv_heads: usize,
    pub head_dim: usize,
    pub seq_len: usize,
    pub max_len: usize,
    pub eps: f32,
    /// The shape record `teeny_flash_attn_fwd_bf16` takes by pointer; rewritten by every `pack_args` and read by the
    /// call that follows it on the same thread.
    shape: Mutex<Box<TeenyAttnShape>>,
}

impl QwenAttention {
    pub const ENTRY_POINTS: [&'static str; 2] = ["teeny_qk_norm_rope_kv_bf16", "teeny_flash_attn_fwd_bf16"];

    pub fn new(num_q_heads: usize, num_kv_heads: usize, seq_len: usize, max_len: usize, eps: f32) -> Self {
        Self { num_q_heads, num_kv_heads, head_dim: 128, seq_len, max_len, eps, shape: Mutex::new(Box::default()) }
    }

    fn qkv_width(&self) -> usize {
        (self.num_q_heads + 2 * self.num_kv_heads) * self.head_dim
    }

    // entry point: teeny_qk_norm_rope_kv_bf16
    fn pack_rope(&self, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], visitor: &mut dyn ArgVisitor) {
        let tokens = inputs[0].1[0];
        visitor.visit_ptr(inputs[0].0); // qkv
        visitor.visit_i64(self.qkv_width() as i64); // ld
        visitor.visit_ptr(params[0]); // q_norm_w
        visitor.visit_ptr(params[1]); // k_norm_w
        visitor.visit_ptr(params[2]); // cos_table
        visitor.visit_ptr(params[3]); // sin_table
        visitor.visit_ptr(params[4]); // k_cache
        visitor.visit_ptr(params[5]); // v_cache
        visitor.visit_i32(tokens as i32); // T
        visitor.visit_i32(self.seq_len as i32); // S
        visitor.visit_i32(self.num_q_heads as i32); // Hq
        visitor.visit_i32(self.num_kv_heads as i32); // Hkv
        visitor.visit_i32(self.head_dim as i32); // D
        visitor.visit_i32(self.max_len as i32); // max_len
        visitor.visit_i32(0); // pos0
        visitor.visit_ptr(core::ptr::null_mut()); // pos0_dev
        visitor.visit_f32(self.eps); // eps
    }

    // entry point: teeny_flash_attn_fwd_bf16
    fn pack_attention(&self, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], output: RawPtr, visitor: &mut dyn ArgVisitor) {
        let (d, hq, hkv) = (self.head_dim as i64, self.num_q_heads as i64, self.num_kv_heads as i64);
        let (s, w) = (self.seq_len as i64, self.qkv_width() as i64);
        let batch = inputs[0].1[0] as i64 / s;
        let mut shape = self.shape.lock().unwrap();
        **shape = TeenyAttnShape {
            b: batch as i32, hq: hq as i32, hkv: hkv as i32, sq: s as i32, skv: s as i32, d: d as i32,
            q_sb: s * w, q_sh: d, q_ss: w,                                   // q read in place inside the projection
            k_sb: hkv * self.max_len as i64 * d, k_sh: self.max_len as i64 * d, k_ss: d,
            v_sb: hkv * self.max_len as i64 * d, v_sh: self.max_len as i64 * d, v_ss: d,
            o_sb: s * hq * d, o_sh: d, o_ss: hq * d,                         // token-major output, what o_proj consumes
            scale: 1.0 / (d as f32).sqrt(), causal: 1,
        };
        visitor.visit_ptr(inputs[0].0); // q
        visitor.visit_ptr(params[4]); // k
        visitor.visit_ptr(params[5]); // v
        visitor.visit_ptr(output); // o
        visitor.visit_ptr(core::ptr::null_mut()); // lse
        visitor.visit_ptr((&mut **shape as *mut TeenyAttnShape).cast()); // shape
    }
}

impl RuntimeOp for QwenAttention {
    fn n_activation_inputs(&self) -> usize {
        1
    }

    fn param_shapes(&self, input_shapes: &[&[usize]], _output_shape: &[usize]) -> Vec<Vec<usize>> {
        let batch = input_shapes[0][0] / self.seq_len;
        let cache = vec![batch, self.num_kv_heads, self.max_len, self.head_dim];
        vec![vec![self.head_dim], vec![self.head_dim], vec![self.max_len, self.head_dim], vec![self.max_len, self.head_dim],
             cache.clone(), cache]
    }

    fn param_names(&self) -> &'static [&'static str] {
        &["q_norm.weight", "k_norm.weight", "rope_cos", "rope_sin", "k_cache", "v_cache"]
    }

    fn pack_args(&self, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], _output: RawPtr, _output_shape: &[usize],
                 _output_row_stride: i32, visitor: &mut dyn ArgVisitor) {
        self.pack_rope(inputs, params, visitor);
    }

    fn n_launches(&self) -> usize {
        2
    }

    fn pack_args_for_launch(&self, launch_idx: usize, inputs: &[(RawPtr, &[usize])], params: &[RawPtr], output: RawPtr,
                            _output_shape: &[usize], _output_row_stride: i32, visitor: &mut dyn ArgVisitor) {
        match launch_idx {
            0 => self.pack_rope(inputs, params, visitor),
            _ => self.pack_attention(inputs, params, output, visitor),
        }
    }

    fn block(&self) -> [u32; 3] {
        ONE_WARP
    }

    fn grid(&self, _output_shape: &[usize]) -> [u32; 3] {
        ONE_CTA
    }
}

impl CustomOp for QwenAttention {
    fn name(&self) -> &str {
        "qwen_attention"
    }

    fn infer_output_shape(&self, input_shapes: &[&Shape]) -> Shape {
        vec![input_shapes[0][0], Some(self.num_q_heads * self.head_dim)]
    }

    fn as_any(&self) -> &dyn Any {
        self
    }

    /// The executor launches `ENTRY_POINTS[i]` for launch `i`; the tuple carries the first.
    fn lower(&self) -> Option<(String, String, String, Arc<dyn RuntimeOp>)> {
        let op = QwenAttention::new(self.num_q_heads, self.num_kv_heads, self.seq_len, self.max_len, self.eps);
        lowered("qwen_attention", Self::ENTRY_POINTS[0], Arc::new(op))
    }
}
