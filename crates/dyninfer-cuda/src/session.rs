//! `ModelSession` of the cuda target: the paged-KV half of
//! `crates/dyninfer-runtime/src/session.rs:88-389` over [`crate::Context`].
//!
//! The cuda target has no static-globals KV mode: the cache is always the paged pool of
//! `configure_paged_kv` (256-token pages, prompt chunks of `chunk_size`), so only that branch of
//! the reference session exists here. Limits, chunking, right padding with the pad id,
//! position tracking and every error message follow the reference, because `generate_greedy`
//! (`crates/dyninfer-runtime/src/generate.rs:117-232`) and `run_perf` (`perf.rs:92-172`) drive
//! this type exactly as they drive `IreeSession`.
//!
//! Not compiled in this repository's build image (no `rustc`).

use crate::Context;
use dyninfer_core::{KvCacheDescriptor, KvCacheStorage, ModelMetadata, SessionConfig, TokenId};
use dyninfer_error::{DynInferError, IreeRuntimeError, Result};
use dyninfer_runtime::{AllocatorMetrics, KvCacheMetrics, Logits, ModelSession};
use std::sync::Arc;
use tracing::info_span;

fn refuse(message: String) -> DynInferError {
    DynInferError::IreeRuntime(IreeRuntimeError { message, status_code: None })
}

pub struct CudaSession {
    metadata: ModelMetadata,
    config: SessionConfig,
    kv: KvCacheDescriptor,
    page_size: usize,
    chunk_size: usize,
    pad_token_id: TokenId,
    position: u64,
    history: Vec<TokenId>,
    context: Arc<Context>,
}

impl CudaSession {
    /// `kv.storage` must be `KvCacheStorage::Paged`; the geometry given to the context's
    /// `configure_paged_kv` must be the same one.
    pub fn new(metadata: ModelMetadata, config: SessionConfig, kv: KvCacheDescriptor, context: Arc<Context>) -> Result<Self> {
        let (page_size, chunk_size) = match kv.storage {
            KvCacheStorage::Paged { page_size, chunk_size } => (page_size as usize, chunk_size as usize),
            KvCacheStorage::StaticGlobals => {
                return Err(refuse("the cuda target keeps its KV cache in a paged pool only".into()));
            }
        };
        let pad_token_id = ["pad_token_id", "bos_token_id"]
            .iter()
            .find_map(|k| metadata.extra.get(*k).and_then(|v| v.as_u64()))
            .map(|v| v as TokenId)
            .unwrap_or(0);
        Ok(Self {
            metadata,
            config,
            kv,
            page_size: page_size.max(1),
            chunk_size: chunk_size.max(1),
            pad_token_id,
            position: 0,
            history: Vec::new(),
            context,
        })
    }

    /// Session limit and cache capacity, whichever is smaller.
    fn max_seq(&self) -> u64 {
        (self.config.max_sequence_length.max(1) as u64).min(self.kv.max_sequence_length.max(1) as u64)
    }

    fn max_pages(&self) -> usize {
        (self.max_seq() as usize).div_ceil(self.page_size).max(1)
    }

    fn require_batch_1(&self) -> Result<()> {
        if self.config.batch_size == 1 {
            Ok(())
        } else {
            Err(refuse(format!(
                "batch_size {} is not supported (only batch_size=1)",
                self.config.batch_size
            )))
        }
    }

    fn check_prompt(&self, tokens: &[TokenId]) -> Result<()> {
        self.require_batch_1()?;
        if tokens.is_empty() {
            return Err(refuse("prefill requires a non-empty token list".into()));
        }
        let limit = self.max_seq() as usize;
        if tokens.len() > limit {
            return Err(refuse(format!(
                "prefill length {} exceeds session/KV limit {}",
                tokens.len(),
                limit
            )));
        }
        Ok(())
    }

    fn check_step(&self) -> Result<()> {
        self.require_batch_1()?;
        // The position is the next write index into the cache: at the limit, refuse.
        if self.position >= self.max_seq() {
            return Err(refuse(format!(
                "decode position {} exceeds session/KV limit {}",
                self.position,
                self.max_seq()
            )));
        }
        Ok(())
    }

    /// One chunk-sized window: the chunk's tokens first, the pad id after them.
    fn window(&self, chunk: &[TokenId]) -> (Vec<i64>, i64) {
        let mut w = vec![i64::from(self.pad_token_id); self.chunk_size];
        for (slot, &t) in w.iter_mut().zip(chunk) {
            *slot = i64::from(t);
        }
        (w, chunk.len().max(1) as i64 - 1)
    }

    /// Feeds the prompt chunk by chunk; logits are fetched for the last chunk only when wanted.
    fn run_prompt(&mut self, tokens: &[TokenId], want_logits: bool) -> Result<(Option<Vec<f32>>, i64)> {
        self.history.clear();
        self.history.extend_from_slice(tokens);
        self.context.reset_paged_kv()?;
        self.context.ensure_kv_pages(self.max_pages())?;
        let chunk_count = tokens.len().div_ceil(self.chunk_size);
        let mut logits = None;
        let mut token = -1i64;
        for (index, chunk) in tokens.chunks(self.chunk_size).enumerate() {
            let (window, last) = self.window(chunk);
            let final_chunk = index + 1 == chunk_count;
            let (l, t) = self.context.invoke_paged_chunk_ex(
                &window,
                last,
                (index * self.chunk_size) as i64,
                want_logits && final_chunk,
            )?;
            if final_chunk {
                logits = l;
            }
            token = t;
        }
        self.position = tokens.len() as u64;
        Ok((logits, token))
    }

    fn check_vocab(&self, what: &str, values: &[f32]) -> Result<()> {
        if values.len() == self.metadata.vocabulary_size as usize {
            Ok(())
        } else {
            Err(refuse(format!(
                "{what} returned {} logits, expected vocab {}",
                values.len(),
                self.metadata.vocabulary_size
            )))
        }
    }
}

impl ModelSession for CudaSession {
    fn prefill(&mut self, tokens: &[TokenId]) -> Result<Logits> {
        let _span = info_span!("runtime.prefill", tokens = tokens.len()).entered();
        self.check_prompt(tokens)?;
        let (logits, _) = self.run_prompt(tokens, true)?;
        let values = logits.ok_or_else(|| refuse("final prefill chunk returned no logits".into()))?;
        self.check_vocab("prefill", &values)?;
        Ok(Logits { values })
    }

    fn decode(&mut self, token: TokenId) -> Result<Logits> {
        let _span = info_span!("runtime.decode", token, position = self.position).entered();
        self.check_step()?;
        self.context.ensure_kv_pages(self.max_pages())?;
        let values = self.context.invoke_paged_chunk(&[i64::from(token)], 0, self.position as i64)?;
        self.check_vocab("decode", &values)?;
        self.history.push(token);
        self.position += 1;
        Ok(Logits { values })
    }

    fn prefill_argmax(&mut self, tokens: &[TokenId]) -> Result<TokenId> {
        let _span = info_span!("runtime.prefill_argmax", tokens = tokens.len()).entered();
        self.check_prompt(tokens)?;
        let (_, token) = self.run_prompt(tokens, false)?;
        if token < 0 {
            return Err(refuse(format!("prefill_argmax returned invalid token {token}")));
        }
        Ok(token as TokenId)
    }

    fn decode_argmax(&mut self, token: TokenId) -> Result<TokenId> {
        let _span = info_span!("runtime.decode_argmax", token, position = self.position).entered();
        self.check_step()?;
        self.context.ensure_kv_pages(self.max_pages())?;
        // 24 bytes in, 8 bytes out: no vocabulary-sized copy on this path.
        let (_, next) = self
            .context
            .invoke_paged_chunk_ex(&[i64::from(token)], 0, self.position as i64, false)?;
        if next < 0 {
            return Err(refuse(format!("decode_argmax returned invalid token {next}")));
        }
        self.history.push(token);
        self.position += 1;
        Ok(next as TokenId)
    }

    fn position(&self) -> u64 {
        self.position
    }

    fn reset(&mut self) -> Result<()> {
        self.context.reset_paged_kv()?; // zero-fills in place; the pool keeps its pages
        self.position = 0;
        self.history.clear();
        Ok(())
    }

    fn kv_cache_metrics(&self) -> Result<KvCacheMetrics> {
        let (page_count, allocated) = self.context.paged_kv_metrics()?;
        Ok(KvCacheMetrics {
            page_count,
            allocated_bytes: allocated,
            capacity_bytes: self.kv.capacity_bytes() as usize,
            used_bytes: allocated,
            filled_tokens: self.position,
            layers: self.kv.layer_count,
            kv_heads: self.kv.kv_head_count,
            head_dim: self.kv.head_dimension,
            max_sequence_length: self.kv.max_sequence_length,
            key_dtype: self.kv.element_type,
            value_dtype: self.kv.element_type,
            paged: true,
            chunk_size: self.chunk_size as u32,
        })
    }

    fn allocator_metrics(&self) -> Result<AllocatorMetrics> {
        let s = self.context.allocator_statistics()?;
        Ok(AllocatorMetrics {
            host_bytes_peak: s.host_bytes_peak,
            host_bytes_allocated: s.host_bytes_allocated,
            host_bytes_freed: s.host_bytes_freed,
            device_bytes_peak: s.device_bytes_peak,
            device_bytes_allocated: s.device_bytes_allocated,
            device_bytes_freed: s.device_bytes_freed,
        })
    }
}
