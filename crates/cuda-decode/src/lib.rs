//! Safe wrapper over the C ABI of `libcuda_decode.so` (include/cuda_decode.h) with the public
//! surface of `metal_decode::Model` (crates/metal-decode/src/lib.rs:129-511): same method names,
//! argument meaning, return values and panics, so `engine::decode::DecodeContext` can switch
//! backend without any other change.  Additive methods (`prefill`, `decode_steps_*`,
//! `from_checkpoint`, tensor parallelism) follow.
//!
//! NOT COMPILED in this repository: the build environment has no Rust toolchain.
use std::ffi::{c_char, c_int, c_void, CStr, CString};

pub const MAX_GPU_TOPK: usize = 32; // lib.rs:15
pub const HEAD_BLOCK: usize = 256; // lib.rs:156

pub const DTYPE_F32: i32 = 0;
pub const DTYPE_F16: i32 = 1;
pub const DTYPE_BF16: i32 = 2;
pub const DTYPE_FP8_E4M3: i32 = 3;
pub const DTYPE_INT4_G32: i32 = 4;
pub const KV_AUTO: i32 = 0;
pub const KV_F32: i32 = 1;
pub const KV_F16: i32 = 2;
pub const KV_BF16: i32 = 3;

/// metal_decode::Config, lib.rs:22-35.
#[repr(C)]
#[derive(Clone, Debug, Default)]
pub struct Config {
    pub dim: i32,
    pub hidden: i32,
    pub heads: i32,
    pub kv_heads: i32,
    pub hd: i32,
    pub seq: i32,
    pub nlayers: i32,
    pub vocab: i32,
    pub q_dim: i32,
    pub kv_dim: i32,
    pub gqa_ratio: i32,
}

/// metal_decode::LayerInit, lib.rs:37-47 (fp32 host tensors in the reference's layouts).
pub struct LayerInit<'a> {
    pub wq: &'a [f32],
    pub wk: &'a [f32],
    pub wv: &'a [f32],
    pub wo: &'a [f32],
    pub w1: &'a [f32],
    pub w3: &'a [f32],
    pub w2: &'a [f32],
    pub gamma1: &'a [f32],
    pub gamma2: &'a [f32],
}

/// metal_decode::FinalHeadInit, lib.rs:49-52; `lm_head: None` is the reference's tied head.
pub struct FinalHeadInit<'a> {
    pub gamma_final: &'a [f32],
    pub embed: &'a [f32],
    pub lm_head: Option<&'a [f32]>,
}

/// cd_options: what the reference has no field for.  `Default` is reference behaviour.
#[repr(C)]
#[derive(Clone, Debug, Default)]
pub struct Options {
    pub weight_dtype: i32,
    pub activation: i32,
    pub device: i32,
    pub page_tokens: i32,
    pub max_samples: i32,
    pub use_graph: i32,
    pub kv_dtype: i32,
    pub tp_rank: i32,
    pub tp_world: i32,
    pub wait_us: i32,
    pub test_flags: i32,
    pub test_ring_kb: i32,
}

#[repr(C)]
struct RawLayerInit {
    wq: *const f32,
    wk: *const f32,
    wv: *const f32,
    wo: *const f32,
    w1: *const f32,
    w3: *const f32,
    w2: *const f32,
    gamma1: *const f32,
    gamma2: *const f32,
}

#[repr(C)]
struct RawHeadInit {
    gamma_final: *const f32,
    embed: *const f32,
    lm_head: *const f32,
}

extern "C" {
    fn cd_model_create(cfg: *const Config, layers: *const RawLayerInit, nlayers: c_int, head: *const RawHeadInit,
                       opts: *const Options, out: *mut *mut c_void) -> c_int;
    fn cd_model_create_from_checkpoint(path: *const c_char, opts: *const Options, cfg_out: *mut Config,
                                       out: *mut *mut c_void) -> c_int;
    fn cd_convert_checkpoint(src: *const c_char, dst: *const c_char, quant_dtype: c_int, device: c_int) -> c_int;
    fn cd_model_destroy(m: *mut c_void);
    fn cd_last_error(m: *const c_void) -> *const c_char;
    fn cd_len(m: *const c_void, len: *mut usize) -> c_int;
    fn cd_set_len(m: *mut c_void, len: usize) -> c_int;
    fn cd_seed_layer_cache_cf(m: *mut c_void, layer: c_int, live_len: usize, k: *const f32, v: *const f32) -> c_int;
    fn cd_decode_token(m: *mut c_void, x_in: *const f32, x_out: *mut f32) -> c_int;
    fn cd_decode_token_from_id(m: *mut c_void, token: u32, x_out: *mut f32) -> c_int;
    fn cd_decode_token_argmax(m: *mut c_void, x_in: *const f32, out: *mut u32) -> c_int;
    fn cd_decode_token_argmax_from_id(m: *mut c_void, token: u32, out: *mut u32) -> c_int;
    fn cd_decode_token_topk_from_id(m: *mut c_void, token: u32, top_k: usize, vals: *mut f32, idxs: *mut u32,
                                    cap: usize, count: *mut usize) -> c_int;
    fn cd_decode_token_block_stats_from_id(m: *mut c_void, token: u32, inv_t: f32, softcap: f32, maxes: *mut f32,
                                           sums: *mut f32, cap: usize, nblocks: *mut usize) -> c_int;
    fn cd_materialize_current_logits_block(m: *mut c_void, block: usize, softcap: f32, out: *mut f32, cap: usize,
                                           valid: *mut usize) -> c_int;
    fn cd_decode_token_logits_from_id(m: *mut c_void, token: u32, softcap: f32, out: *mut f32) -> c_int;
    fn cd_prefill(m: *mut c_void, ids: *const u32, n: usize, softcap: f32, last_logits: *mut f32) -> c_int;
    fn cd_decode_steps_greedy(m: *mut c_void, first: u32, nsteps: usize, out_ids: *mut u32) -> c_int;
    fn cd_decode_steps_topk(m: *mut c_void, first: u32, nsteps: usize, top_k: usize, t: f32, softcap: f32,
                            rng: *mut u64, out_ids: *mut u32) -> c_int;
    fn cd_decode_steps_fullvocab(m: *mut c_void, first: u32, nsteps: usize, t: f32, softcap: f32, rng: *mut u64,
                                 out_ids: *mut u32) -> c_int;
    fn cd_decode_steps_samples(m: *mut c_void, first: *const u32, nsamples: usize, nsteps: usize, mode: c_int,
                               top_k: usize, t: f32, softcap: f32, rng: *mut u64, out_ids: *mut u32) -> c_int;
    fn cd_tp_region_handle(m: *mut c_void, out: *mut c_void, cap: usize) -> c_int;
    fn cd_tp_connect(m: *mut c_void, handles: *const c_void, world: c_int) -> c_int;
}

/// A KV-cached single-token decoder resident on one B200 (`metal_decode::Model`, lib.rs:129-144).
pub struct Model {
    h: *mut c_void,
    cfg: Config,
    argmax_blocks: usize,
}

// The handle owns device memory and a stream; it may move between threads but is used by one at a
// time (`&mut self` on every call, as the reference).
unsafe impl Send for Model {}

fn global_error() -> String {
    unsafe { CStr::from_ptr(cd_last_error(std::ptr::null())) }.to_string_lossy().into_owned()
}

impl Model {
    /// Model::new, lib.rs:147-207: `None` on any construction failure.
    pub fn new<'a>(cfg: &Config, layers: impl IntoIterator<Item = LayerInit<'a>>, final_head: FinalHeadInit<'a>)
                   -> Option<Self> {
        Self::new_with_options(cfg, layers, final_head, &Options { device: -1, ..Options::default() })
    }

    pub fn new_with_options<'a>(cfg: &Config, layers: impl IntoIterator<Item = LayerInit<'a>>,
                                final_head: FinalHeadInit<'a>, opts: &Options) -> Option<Self> {
        let raw: Vec<RawLayerInit> = layers
            .into_iter()
            .map(|l| RawLayerInit {
                wq: l.wq.as_ptr(), wk: l.wk.as_ptr(), wv: l.wv.as_ptr(), wo: l.wo.as_ptr(), w1: l.w1.as_ptr(),
                w3: l.w3.as_ptr(), w2: l.w2.as_ptr(), gamma1: l.gamma1.as_ptr(), gamma2: l.gamma2.as_ptr(),
            })
            .collect();
        let head = RawHeadInit {
            gamma_final: final_head.gamma_final.as_ptr(),
            embed: final_head.embed.as_ptr(),
            lm_head: final_head.lm_head.map_or(std::ptr::null(), |s| s.as_ptr()),
        };
        let mut out = std::ptr::null_mut();
        let rc = unsafe { cd_model_create(cfg, raw.as_ptr(), raw.len() as c_int, &head, opts, &mut out) };
        if rc != 0 {
            return None;
        }
        Some(Self::wrap(out, cfg.clone()))
    }

    /// Streams an RSTK checkpoint (checkpoint.rs:25-209 formats, plus the v3 header) into HBM.
    pub fn from_checkpoint(path: &str, opts: &Options) -> Result<Self, String> {
        let c = CString::new(path).map_err(|e| e.to_string())?;
        let (mut cfg, mut out) = (Config::default(), std::ptr::null_mut());
        let rc = unsafe { cd_model_create_from_checkpoint(c.as_ptr(), opts, &mut cfg, &mut out) };
        if rc != 0 {
            return Err(global_error());
        }
        Ok(Self::wrap(out, cfg))
    }

    /// Quantises the linears of an RSTK file once (`quant_dtype` 3: FP8-E4M3 with a scale per output row,
    /// 4: INT4 in groups of 32) and writes an RSTK v3 file that `from_checkpoint` streams into HBM as it is.
    pub fn convert_checkpoint(src: &str, dst: &str, quant_dtype: i32, device: i32) -> Result<(), String> {
        let (s, d) = (CString::new(src).map_err(|e| e.to_string())?, CString::new(dst).map_err(|e| e.to_string())?);
        let rc = unsafe { cd_convert_checkpoint(s.as_ptr(), d.as_ptr(), quant_dtype, device) };
        if rc != 0 {
            return Err(global_error());
        }
        Ok(())
    }

    fn wrap(h: *mut c_void, cfg: Config) -> Self {
        let argmax_blocks = (cfg.vocab as usize + HEAD_BLOCK - 1) / HEAD_BLOCK;
        Self { h, cfg, argmax_blocks }
    }

    /// The reference asserts; the panic and its message are kept.
    fn check(&self, rc: c_int) {
        if rc != 0 {
            panic!("{}", unsafe { CStr::from_ptr(cd_last_error(self.h)) }.to_string_lossy());
        }
    }

    fn fallible(&self, rc: c_int) -> Result<(), String> {
        if rc == 0 {
            Ok(())
        } else {
            Err(unsafe { CStr::from_ptr(cd_last_error(self.h)) }.to_string_lossy().into_owned())
        }
    }

    pub fn config(&self) -> &Config {
        &self.cfg
    }

    /// lib.rs:209
    pub fn len(&self) -> usize {
        let mut n = 0usize;
        self.check(unsafe { cd_len(self.h, &mut n) });
        n
    }

    /// lib.rs:211-215 (clamped to seq)
    pub fn set_len(&mut self, len: usize) {
        self.check(unsafe { cd_set_len(self.h, len) })
    }

    /// lib.rs:217-237: `k_rope_cf` and `v_cf` are channel-first `[kv_dim, seq]`.
    pub fn seed_layer_cache_from_channel_first(&mut self, layer_idx: usize, live_len: usize, k_rope_cf: &[f32],
                                               v_cf: &[f32]) {
        let need = self.cfg.kv_dim as usize * self.cfg.seq as usize;
        assert!(k_rope_cf.len() >= need && v_cf.len() >= need, "k_rope_cf / v_cf must hold kv_dim * seq values");
        self.check(unsafe {
            cd_seed_layer_cache_cf(self.h, layer_idx as c_int, live_len, k_rope_cf.as_ptr(), v_cf.as_ptr())
        })
    }

    /// lib.rs:239-269
    pub fn decode_token(&mut self, x_in: &[f32], x_out: &mut [f32]) {
        assert_eq!(x_in.len(), self.cfg.dim as usize);
        assert_eq!(x_out.len(), self.cfg.dim as usize);
        self.check(unsafe { cd_decode_token(self.h, x_in.as_ptr(), x_out.as_mut_ptr()) })
    }

    /// lib.rs:271-304
    pub fn decode_token_from_id(&mut self, token: u32, x_out: &mut [f32]) {
        assert_eq!(x_out.len(), self.cfg.dim as usize);
        self.check(unsafe { cd_decode_token_from_id(self.h, token, x_out.as_mut_ptr()) })
    }

    /// lib.rs:306-338
    pub fn decode_token_argmax(&mut self, x_in: &[f32]) -> u32 {
        assert_eq!(x_in.len(), self.cfg.dim as usize);
        let mut out = 0u32;
        self.check(unsafe { cd_decode_token_argmax(self.h, x_in.as_ptr(), &mut out) });
        out
    }

    /// lib.rs:340-375
    pub fn decode_token_argmax_from_id(&mut self, token: u32) -> u32 {
        let mut out = 0u32;
        self.check(unsafe { cd_decode_token_argmax_from_id(self.h, token, &mut out) });
        out
    }

    /// lib.rs:377-434: writes `nblocks * top_k` (value, index) pairs block-major; returns that count.
    pub fn decode_token_topk_from_id(&mut self, token: u32, top_k: usize, out_vals: &mut [f32], out_idxs: &mut [u32])
                                     -> usize {
        let cap = out_vals.len().min(out_idxs.len());
        let mut n = 0usize;
        self.check(unsafe {
            cd_decode_token_topk_from_id(self.h, token, top_k, out_vals.as_mut_ptr(), out_idxs.as_mut_ptr(), cap, &mut n)
        });
        n
    }

    /// lib.rs:436-487: returns the number of blocks.
    pub fn decode_token_block_stats_from_id(&mut self, token: u32, inv_temperature: f32, softcap: f32,
                                            out_maxes: &mut [f32], out_sums: &mut [f32]) -> usize {
        let cap = out_maxes.len().min(out_sums.len());
        let mut n = 0usize;
        self.check(unsafe {
            cd_decode_token_block_stats_from_id(self.h, token, inv_temperature, softcap, out_maxes.as_mut_ptr(),
                                                out_sums.as_mut_ptr(), cap, &mut n)
        });
        n
    }

    /// lib.rs:489-511: does not advance `len`; returns the number of valid logits (<= 256).
    pub fn materialize_current_logits_block(&mut self, block_idx: usize, softcap: f32, out_logits: &mut [f32]) -> usize {
        let mut n = 0usize;
        self.check(unsafe {
            cd_materialize_current_logits_block(self.h, block_idx, softcap, out_logits.as_mut_ptr(), out_logits.len(),
                                                &mut n)
        });
        n
    }

    pub fn argmax_blocks(&self) -> usize {
        self.argmax_blocks
    }

    // ---- additive: the token loop on the device ------------------------------------------------

    /// DecodeContext::decode_next_logits (decode.rs:91-127) with the final norm and LM head on the GPU.
    pub fn decode_token_logits_from_id(&mut self, token: u32, softcap: f32, out_logits: &mut [f32]) {
        assert_eq!(out_logits.len(), self.cfg.vocab as usize);
        self.check(unsafe { cd_decode_token_logits_from_id(self.h, token, softcap, out_logits.as_mut_ptr()) })
    }

    /// Prompt (or prompt-suffix) pass starting at the cached length; replaces the forward pass of
    /// InferenceSession::new (inference.rs:124-161) and prefill_prompt_suffix_cached (:650-670).
    pub fn prefill(&mut self, ids: &[u32], softcap: f32, last_logits: Option<&mut [f32]>) -> Result<(), String> {
        let p = last_logits.map_or(std::ptr::null_mut(), |s| s.as_mut_ptr());
        self.fallible(unsafe { cd_prefill(self.h, ids.as_ptr(), ids.len(), softcap, p) })
    }

    /// run_cached_sample's greedy loop (inference.rs:576-585) without a host round trip per token.
    pub fn decode_steps_greedy(&mut self, first_token: u32, nsteps: usize) -> Result<Vec<u32>, String> {
        let mut out = vec![0u32; nsteps];
        self.fallible(unsafe { cd_decode_steps_greedy(self.h, first_token, nsteps, out.as_mut_ptr()) })?;
        Ok(out)
    }

    /// inference.rs:586-599 on the device; `rng` is the sample's LCG state (inference.rs:759).
    pub fn decode_steps_topk(&mut self, first_token: u32, nsteps: usize, top_k: usize, temperature: f32, softcap: f32,
                             rng: &mut u64) -> Result<Vec<u32>, String> {
        let mut out = vec![0u32; nsteps];
        self.fallible(unsafe {
            cd_decode_steps_topk(self.h, first_token, nsteps, top_k, temperature, softcap, rng, out.as_mut_ptr())
        })?;
        Ok(out)
    }

    /// inference.rs:600-625 on the device (block statistics, block draw, token draw).
    pub fn decode_steps_fullvocab(&mut self, first_token: u32, nsteps: usize, temperature: f32, softcap: f32,
                                  rng: &mut u64) -> Result<Vec<u32>, String> {
        let mut out = vec![0u32; nsteps];
        self.fallible(unsafe {
            cd_decode_steps_fullvocab(self.h, first_token, nsteps, temperature, softcap, rng, out.as_mut_ptr())
        })?;
        Ok(out)
    }

    /// `--samples N` sharing the cached prompt (inference.rs:255-297 runs them one after the other).
    /// mode: 0 greedy, 1 top-k, 2 full vocabulary.  Returns ids `[nsamples][nsteps]`.
    pub fn decode_steps_samples(&mut self, first_tokens: &[u32], nsteps: usize, mode: i32, top_k: usize, temperature: f32,
                                softcap: f32, rng_states: &mut [u64]) -> Result<Vec<u32>, String> {
        assert_eq!(first_tokens.len(), rng_states.len());
        let mut out = vec![0u32; first_tokens.len() * nsteps];
        self.fallible(unsafe {
            cd_decode_steps_samples(self.h, first_tokens.as_ptr(), first_tokens.len(), nsteps, mode, top_k, temperature,
                                    softcap, rng_states.as_mut_ptr(), out.as_mut_ptr())
        })?;
        Ok(out)
    }

    // ---- additive: tensor parallelism (one process per GPU) --------------------------------------

    /// The 64-byte CUDA IPC handle of this rank's link region (exchange by any transport).
    pub fn tp_region_handle(&mut self) -> Result<[u8; 64], String> {
        let mut buf = [0u8; 64];
        self.fallible(unsafe { cd_tp_region_handle(self.h, buf.as_mut_ptr() as *mut c_void, 64) })?;
        Ok(buf)
    }

    /// `handles`: every rank's handle, in rank order.
    pub fn tp_connect(&mut self, handles: &[[u8; 64]]) -> Result<(), String> {
        self.fallible(unsafe { cd_tp_connect(self.h, handles.as_ptr() as *const c_void, handles.len() as c_int) })
    }
}

impl Drop for Model {
    fn drop(&mut self) {
        unsafe { cd_model_destroy(self.h) }
    }
}
