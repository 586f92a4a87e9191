//! `ferrum_cuda` — Ferrum's quantized transformer forward path on one or more NVIDIA B200 GPUs.
//!
//! Mirrors the numeric surface of `ferrum_core`: `GenerativeSLM::{score, score_rolling, evaluate_ids,
//! token_logprobs, generate_tokens}` (slm/scoring.rs, slm/token_stream.rs), `CachedTransformer::{prime, feed}`
//! (slm/cached.rs) and the wasm `TransformerSLMModel::{predict_next, prime, predict_next_cached, cached_len}`
//! (slm_wasm/src/lib.rs:217-241), on token ids. Text, tokenizer, chat templates and stop strings stay in
//! `ferrum_core`. There is no CPU fallback: construction fails when no sm_100 device is visible.
//!
//! Threading follows the reference: a model is used from one thread at a time (`GenerativeSLM` is `!Send`
//! because of its `RefCell`, layer/transformer.rs:82; the server keeps it on a dedicated thread,
//! slm_server/src/model_thread.rs:111-143). The handles here are `!Send` / `!Sync` for the same reason.
//!
//! This crate was written without a Rust toolchain at hand and has not been compiled; `ffi.rs` is checked
//! against the C header by a test of the CUDA repository.
pub mod ffi;

use std::ffi::{CStr, CString};
use std::marker::PhantomData;
use std::os::raw::c_int;
use std::ptr;
use std::sync::atomic::AtomicBool;

use ferrum_core::error::{InferError, Result};
use ferrum_core::slm::Score;

/// The last error text of the calling thread, mapped onto the reference's error enum (error.rs:6-26).
fn status(rc: c_int) -> Result<()> {
    if rc == ffi::FC_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(ffi::fc_last_error()) }.to_string_lossy().into_owned();
    Err(match rc {
        ffi::FC_E_SHAPE => InferError::ShapeMismatch,
        ffi::FC_E_DIM => InferError::DimMismatch(msg),
        ffi::FC_E_FORMAT => InferError::Format(msg),
        // no variant of the reference's enum names a device: carry the text
        _ => InferError::DimMismatch(format!("ferrum_cuda status {rc}: {msg}")),
    })
}

fn ids32(ids: &[usize]) -> Vec<i32> {
    ids.iter().map(|&i| i32::try_from(i).unwrap_or(i32::MAX)).collect()   // ids past i32 are out of every vocabulary: FC_E_DIM
}

/// Math mode of the window forward (scoring, prime): exact fp32 CUDA cores, or tcgen05 tensor cores on a
/// three-term bf16 split of the f32 operands (2^-16 relative per product). Decode is fp32-equivalent in both.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum MathMode { Fp32 = 0, Bf16x3 = 1 }

/// Decoding controls of slm/sampling.rs:26-39.
pub use ffi::fc_sampling as Sampling;

/// A gpt2-architecture Q8_0 model resident on one GPU (`Sequential` + weights, model.rs:51-71).
pub struct CudaModel {
    raw: *mut ffi::fc_model,
    _not_send: PhantomData<*mut ()>,
}

impl CudaModel {
    /// Straight from a GGUF file, the matrices uploaded as stored (no f32 expansion, the path
    /// loader/decode.rs:99-100 leaves open). `row_perm[model id] = row of the file` is the tokenizer's
    /// permutation (loader/gpt2.rs:221-231); pass `None` when the file's order is the tokenizer's.
    pub fn from_gguf(path: &str, row_perm: Option<&[i32]>, device: usize, math: MathMode) -> Result<Self> {
        let c = CString::new(path).map_err(|_| InferError::Format("path contains a NUL byte".into()))?;
        let (p, n) = row_perm.map_or((ptr::null(), 0), |r| (r.as_ptr(), r.len() as c_int));
        let mut raw = ptr::null_mut();
        status(unsafe { ffi::fc_model_load_gguf(c.as_ptr(), p, n, device as c_int, math as c_int, &mut raw) })?;
        Ok(Self { raw, _not_send: PhantomData })
    }

    /// From tensors already in memory in GGUF order (loader/gpt2.rs:236-262): raw Q8_0 blocks for the
    /// matrices (re-encode Ferrum's f32 `Linear`s with `quant::q8_0_block` along the input dimension; snapped
    /// values re-encode to the same bytes, quant.rs:346-354), f32 slices for everything else. The library
    /// copies during the call; the borrowed buffers may be dropped afterwards.
    ///
    /// # Safety
    /// Every pointer of `weights` must be valid for the extent `cfg` implies.
    pub unsafe fn from_tensors(cfg: &ffi::fc_config, weights: &ffi::fc_weights, device: usize) -> Result<Self> {
        let mut raw = ptr::null_mut();
        status(ffi::fc_model_create(cfg, weights, device as c_int, &mut raw))?;
        Ok(Self { raw, _not_send: PhantomData })
    }

    pub fn config(&self) -> Result<ffi::fc_config> {
        let mut c = ffi::fc_config::default();
        status(unsafe { ffi::fc_model_config(self.raw, &mut c) })?;
        Ok(c)
    }

    /// `GenerativeSLM::token_logprobs` (scoring.rs:151-213) summed into a `Score`.
    pub fn score_from(&self, ids: &[usize], from: usize) -> Result<Score> {
        let v = ids32(ids);
        let mut s = ffi::fc_score::default();
        status(unsafe { ffi::fc_token_logprobs(self.raw, v.as_ptr(), v.len() as c_int, from as c_int, &mut s, ptr::null_mut(), ptr::null_mut()) })?;
        Ok(Score { logprob: s.logprob, n_tokens: s.n_tokens as usize, greedy: s.greedy != 0 })
    }
    /// `GenerativeSLM::score(ctx, cont)` (scoring.rs:95-131) on ids.
    pub fn score(&self, ctx: &[usize], cont: &[usize]) -> Result<Score> {
        let all: Vec<usize> = ctx.iter().chain(cont).copied().collect();
        self.score_from(&all, ctx.len())
    }
    /// `score_rolling` / `evaluate_ids` (scoring.rs:136-140, 77-87).
    pub fn evaluate_ids(&self, ids: &[usize]) -> Result<Score> { self.score_from(ids, 1) }

    /// Many requests in shared forward passes (the model thread of the server scores them one by one,
    /// model_thread.rs:29-38): request r is `ids[offsets[r]..offsets[r + 1]]` scored from `from[r]`.
    pub fn score_requests(&self, ids: &[i32], offsets: &[i64], from: &[i32]) -> Result<Vec<Score>> {
        let n = from.len();
        let mut out = vec![ffi::fc_score::default(); n];
        status(unsafe { ffi::fc_score_requests(self.raw, ids.as_ptr(), offsets.as_ptr(), from.as_ptr(), n as c_int, 0, out.as_mut_ptr()) })?;
        Ok(out.iter().map(|s| Score { logprob: s.logprob, n_tokens: s.n_tokens as usize, greedy: s.greedy != 0 }).collect())
    }

    /// wasm `predict_next` (slm_wasm/src/lib.rs:217-241): the distribution after the last of `ids`.
    pub fn predict_next(&self, ids: &[usize]) -> Result<Vec<f32>> {
        let v = ids32(ids);
        let mut probs = vec![0f32; self.config()?.vocab as usize];
        status(unsafe { ffi::fc_predict_next(self.raw, v.as_ptr(), v.len() as c_int, probs.as_mut_ptr()) })?;
        Ok(probs)
    }

    /// Independent greedy generations in lock step (every Q8_0 matrix is read once per step for all of them):
    /// `prompts` is `[n][prompt_len]`; returns the tokens of each stream.
    pub fn decode_batch(&self, prompts: &[i32], prompt_len: usize, max_new: usize, eos: Option<usize>) -> Result<Vec<Vec<i32>>> {
        let n = prompts.len() / prompt_len.max(1);
        let mut out = vec![0i32; n * max_new.max(1)];
        let mut n_out = vec![0 as c_int; n];
        status(unsafe {
            ffi::fc_decode_batch(self.raw, n as c_int, prompts.as_ptr(), prompt_len as c_int, max_new as c_int,
                                 eos.map_or(-1, |e| e as i32), out.as_mut_ptr(), n_out.as_mut_ptr())
        })?;
        Ok((0..n).map(|i| out[i * max_new..i * max_new + n_out[i] as usize].to_vec()).collect())
    }

    /// A KV-cached stream on this model (`CachedTransformer::try_new`, cached.rs:45-64).
    pub fn stream(&self) -> Result<CudaStream<'_>> {
        let mut raw = ptr::null_mut();
        status(unsafe { ffi::fc_stream_create(self.raw, &mut raw) })?;
        Ok(CudaStream { raw, vocab: self.config()?.vocab as usize, _model: PhantomData })
    }

    pub(crate) fn raw(&self) -> *mut ffi::fc_model { self.raw }
}

impl Drop for CudaModel {
    fn drop(&mut self) { unsafe { ffi::fc_model_free(self.raw) } }
}

/// `CachedTransformer` (cached.rs): per-layer KV caches and a position, borrowed from its model.
pub struct CudaStream<'m> {
    raw: *mut ffi::fc_stream,
    vocab: usize,
    _model: PhantomData<&'m CudaModel>,
}

impl CudaStream<'_> {
    pub fn reset(&mut self) -> Result<()> { status(unsafe { ffi::fc_stream_reset(self.raw) }) }
    pub fn cached_len(&self) -> usize { unsafe { ffi::fc_cached_len(self.raw) as usize } }
    /// cached.rs:129-136.
    pub fn prime(&mut self, ids: &[usize]) -> Result<Vec<f32>> {
        let v = ids32(ids);
        let mut p = vec![0f32; self.vocab];
        status(unsafe { ffi::fc_prime(self.raw, v.as_ptr(), v.len() as c_int, p.as_mut_ptr()) })?;
        Ok(p)
    }
    /// cached.rs:100-125: probabilities of the next token.
    pub fn feed(&mut self, token: usize) -> Result<Vec<f32>> {
        let mut p = vec![0f32; self.vocab];
        status(unsafe { ffi::fc_feed(self.raw, token as i32, p.as_mut_ptr()) })?;
        Ok(p)
    }
    /// token_stream.rs:66-189 with temperature <= 0. `cancel` is polled between launches of at most 32 tokens;
    /// a cancelled generation returns the tokens made so far, as the reference does.
    pub fn generate_greedy(&mut self, prompt: &[usize], max_new: usize, eos: Option<usize>, cancel: &AtomicBool) -> Result<Vec<usize>> {
        let v = ids32(prompt);
        let mut out = vec![0i32; max_new.max(1)];
        let mut n: c_int = 0;
        // AtomicBool has the layout of a byte; the library polls a 32-bit word, so the flag is mirrored
        let flag = std::sync::atomic::AtomicI32::new(0);
        let _watch = MirrorFlag::new(cancel, &flag);
        let rc = unsafe {
            ffi::fc_generate_greedy(self.raw, v.as_ptr(), v.len() as c_int, max_new as c_int, eos.map_or(-1, |e| e as i32),
                                    flag.as_ptr() as *const i32, out.as_mut_ptr(), &mut n)
        };
        if rc != ffi::FC_E_CANCELLED { status(rc)?; }
        Ok(out[..n as usize].iter().map(|&t| t as usize).collect())
    }
    /// `generate_tokens` with a sampler (sampling.rs:124-210). `rng_state` is `Rng::state()` going in and the
    /// value for `Rng::from_state` coming out (rng.rs:18-27).
    pub fn generate_sampled(&mut self, prompt: &[usize], max_new: usize, eos: Option<usize>, params: &Sampling, rng_state: &mut u64) -> Result<Vec<usize>> {
        let v = ids32(prompt);
        let mut out = vec![0i32; max_new.max(1)];
        let mut n: c_int = 0;
        status(unsafe {
            ffi::fc_generate_sampled(self.raw, v.as_ptr(), v.len() as c_int, max_new as c_int, eos.map_or(-1, |e| e as i32), params,
                                     rng_state, ptr::null(), out.as_mut_ptr(), &mut n)
        })?;
        Ok(out[..n as usize].iter().map(|&t| t as usize).collect())
    }
}

impl Drop for CudaStream<'_> {
    fn drop(&mut self) { unsafe { ffi::fc_stream_free(self.raw) } }
}

/// Copies an `AtomicBool` into the 32-bit word the library polls, from a helper thread, until dropped.
struct MirrorFlag { stop: std::sync::Arc<AtomicBool>, handle: Option<std::thread::JoinHandle<()>> }
impl MirrorFlag {
    fn new(src: &AtomicBool, dst: &std::sync::atomic::AtomicI32) -> Self {
        use std::sync::atomic::Ordering::Relaxed;
        let stop = std::sync::Arc::new(AtomicBool::new(false));
        let (s, d, st) = (src as *const AtomicBool as usize, dst as *const std::sync::atomic::AtomicI32 as usize, stop.clone());
        // the borrowed flags outlive the helper: it is joined in drop, before either reference ends
        let handle = std::thread::spawn(move || {
            let (s, d) = unsafe { (&*(s as *const AtomicBool), &*(d as *const std::sync::atomic::AtomicI32)) };
            while !st.load(Relaxed) {
                if s.load(Relaxed) { d.store(1, Relaxed); }
                std::thread::sleep(std::time::Duration::from_millis(1));
            }
        });
        Self { stop, handle: Some(handle) }
    }
}
impl Drop for MirrorFlag {
    fn drop(&mut self) {
        self.stop.store(true, std::sync::atomic::Ordering::Relaxed);
        if let Some(h) = self.handle.take() { let _ = h.join(); }
    }
}

/// Weight precision of an imported decoder, as `Gguf::load_llama(kind)` / `load_llama_prec(None)` choose it
/// (gguf/llama.rs:164-176): the file's own blocks brought to Q8_0 (the fast path of this crate), every Linear
/// re-packed to a per-input-row int8 / int4 `QWeight` and run by `ops::qlinear` (what `load_llama(kind)` computes), or
/// `Native`: every matrix kept in the file's block format and decoded inside the kernels (what `load_llama_prec(None)`
/// computes, at the file's footprint).
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum LlamaWeights { AsStored, PackedInt8, PackedInt4, Native }

/// A llama / qwen2 architecture model resident on one GPU: `LlamaModel` of llm.rs:549-565.
pub struct CudaLlama {
    raw: *mut ffi::fc_llama,
    vocab: usize,
    _not_send: PhantomData<*mut ()>,
}

impl CudaLlama {
    /// `Gguf::open(path)?.load_llama(..)` (gguf/llama.rs:164-339) straight from the file to the device.
    pub fn from_gguf(path: &str, device: usize, math: MathMode, ctx_cap: usize, weights: LlamaWeights) -> Result<Self> {
        let c_path = CString::new(path).map_err(|_| InferError::Format("path holds a NUL byte".into()))?;
        let mut cfg: ffi::fc_llama_config = unsafe { std::mem::zeroed() };
        status(unsafe { ffi::fc_llama_gguf_probe(c_path.as_ptr(), &mut cfg) })?;
        let mut raw = ptr::null_mut();
        let (dev, cap) = (device as c_int, ctx_cap as c_int);
        status(match weights {
            LlamaWeights::AsStored => unsafe { ffi::fc_llama_load_gguf(c_path.as_ptr(), dev, math as c_int, cap, &mut raw) },
            LlamaWeights::PackedInt8 => unsafe { ffi::fc_llama_load_gguf_packed(c_path.as_ptr(), dev, cap, ffi::FC_Q_INT8, &mut raw) },
            LlamaWeights::PackedInt4 => unsafe { ffi::fc_llama_load_gguf_packed(c_path.as_ptr(), dev, cap, ffi::FC_Q_INT4, &mut raw) },
            LlamaWeights::Native => unsafe { ffi::fc_llama_load_gguf_native(c_path.as_ptr(), dev, cap, &mut raw) },
        })?;
        Ok(Self { raw, vocab: cfg.vocab as usize, _not_send: PhantomData })
    }

    /// `LlamaModel::forward_tokens` (llm.rs:622-635): logits `[ids.len()][vocab]`, row-major.
    pub fn forward_tokens(&self, ids: &[usize]) -> Result<Vec<f32>> {
        let ids = ids32(ids);
        let mut logits = vec![0f32; ids.len() * self.vocab];
        status(unsafe { ffi::fc_llama_forward_tokens(self.raw, ids.as_ptr(), ids.len() as c_int, logits.as_mut_ptr()) })?;
        Ok(logits)
    }

    /// `LlamaModel::score_from` (llm_score.rs:76-96): the log-probability of `ids[from..]` given what precedes it,
    /// in windows of `window` tokens.
    pub fn score_from(&self, ids: &[usize], from: usize, window: usize) -> Result<Score> {
        let ids = ids32(ids);
        let mut sc: ffi::fc_score = unsafe { std::mem::zeroed() };
        status(unsafe {
            ffi::fc_llama_score_from(self.raw, ids.as_ptr(), ids.len() as c_int, from as c_int, window as c_int, &mut sc,
                                     ptr::null_mut(), ptr::null_mut())
        })?;
        Ok(Score { logprob: sc.logprob, n_tokens: sc.n_tokens as usize, greedy: sc.greedy != 0 })
    }

    /// `LlamaModel::score_rolling` (llm_score.rs:61-69).
    pub fn score_rolling(&self, ids: &[usize], window: usize) -> Result<Score> { self.score_from(ids, 1, window) }
}

impl Drop for CudaLlama {
    fn drop(&mut self) { unsafe { ffi::fc_llama_free(self.raw) } }
}


/// One model per GPU behind a single call: sequences (or decode streams) are split in contiguous blocks and
/// each block runs on its own host thread inside the library; results land in order, nothing is gathered.
pub struct CudaModelSet { models: Vec<CudaModel> }

impl CudaModelSet {
    pub fn new(models: Vec<CudaModel>) -> Self { Self { models } }
    pub fn score_sequences(&self, ids: &[i32], seq_len: usize) -> Result<Vec<Score>> {
        let n = ids.len() / seq_len.max(1);
        let raws: Vec<*mut ffi::fc_model> = self.models.iter().map(|m| m.raw()).collect();
        let mut out = vec![ffi::fc_score::default(); n];
        status(unsafe {
            ffi::fc_score_sequences_multi(raws.as_ptr(), raws.len() as c_int, ids.as_ptr(), n as c_int, seq_len as c_int, 0,
                                          out.as_mut_ptr(), ptr::null_mut())
        })?;
        Ok(out.iter().map(|s| Score { logprob: s.logprob, n_tokens: s.n_tokens as usize, greedy: s.greedy != 0 }).collect())
    }
}
