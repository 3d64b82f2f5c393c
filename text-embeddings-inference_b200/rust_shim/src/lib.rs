//! `Backend` implementation over the C ABI of libtei_b200.so (include/tei_b200.h).
//!
//! Mirrors `CandleBackend` (backends/candle/src/lib.rs:163-168, 639-726): same constructor
//! arguments, same `Embeddings` / `Predictions` maps, same error mapping, so `init_backend`
//! (backends/src/lib.rs:443-607) can select it behind a cargo feature.
use nohash_hasher::BuildNoHashHasher;
use std::collections::HashMap;
use std::ffi::{c_char, c_int, CStr, CString};
use std::path::Path;
use text_embeddings_backend_core::{
    Backend, BackendError, Batch, Embedding, Embeddings, ModelType, Pool, Predictions,
};

#[repr(C)]
struct TeiB200 {
    _private: [u8; 0],
}

extern "C" {
    fn tei_b200_create(
        model_dir: *const c_char,
        dtype: *const c_char,
        model_type: c_int,
        pool: c_int,
        devices: *const c_int,
        n_devices: c_int,
        out: *mut *mut TeiB200,
        err: *mut c_char,
        err_cap: usize,
    ) -> c_int;
    fn tei_b200_add_dense(
        h: *mut TeiB200,
        dense_path: *const c_char,
        err: *mut c_char,
        err_cap: usize,
    ) -> c_int;
    fn tei_b200_destroy(h: *mut TeiB200);
    fn tei_b200_health(h: *mut TeiB200) -> c_int;
    fn tei_b200_is_padded(h: *const TeiB200) -> c_int;
    fn tei_b200_max_batch_size(h: *const TeiB200) -> c_int;
    fn tei_b200_output_dim(h: *const TeiB200) -> c_int;
    fn tei_b200_hidden_size(h: *const TeiB200) -> c_int;
    fn tei_b200_num_classes(h: *const TeiB200) -> c_int;
    fn tei_b200_embed(
        h: *mut TeiB200,
        input_ids: *const u32,
        token_type_ids: *const u32,
        position_ids: *const u32,
        n_tokens: usize,
        cumulative_seq_lengths: *const u32,
        n_seqs: usize,
        max_length: u32,
        pooled_idx: *const u32,
        n_pooled: usize,
        raw_idx: *const u32,
        n_raw: usize,
        normalize: c_int,
        pooled_out: *mut f32,
        raw_out: *mut f32,
        err: *mut c_char,
        err_cap: usize,
    ) -> c_int;
    fn tei_b200_predict(
        h: *mut TeiB200,
        input_ids: *const u32,
        token_type_ids: *const u32,
        position_ids: *const u32,
        n_tokens: usize,
        cumulative_seq_lengths: *const u32,
        n_seqs: usize,
        max_length: u32,
        scores_out: *mut f32,
        err: *mut c_char,
        err_cap: usize,
    ) -> c_int;
    fn tei_b200_num_replicas(h: *const TeiB200) -> c_int;
    fn tei_b200_embed_on(
        h: *mut TeiB200,
        replica: c_int,
        input_ids: *const u32,
        token_type_ids: *const u32,
        position_ids: *const u32,
        n_tokens: usize,
        cumulative_seq_lengths: *const u32,
        n_seqs: usize,
        max_length: u32,
        pooled_idx: *const u32,
        n_pooled: usize,
        raw_idx: *const u32,
        n_raw: usize,
        normalize: c_int,
        pooled_out: *mut f32,
        raw_out: *mut f32,
        err: *mut c_char,
        err_cap: usize,
    ) -> c_int;
    fn tei_b200_predict_on(
        h: *mut TeiB200,
        replica: c_int,
        input_ids: *const u32,
        token_type_ids: *const u32,
        position_ids: *const u32,
        n_tokens: usize,
        cumulative_seq_lengths: *const u32,
        n_seqs: usize,
        max_length: u32,
        scores_out: *mut f32,
        err: *mut c_char,
        err_cap: usize,
    ) -> c_int;
}

const ERR_CAP: usize = 1024;

fn to_error(code: c_int, buf: &[c_char]) -> BackendError {
    let msg = unsafe { CStr::from_ptr(buf.as_ptr()) }
        .to_string_lossy()
        .into_owned();
    match code {
        1 => BackendError::Start(msg),
        3 => BackendError::Unhealthy,
        4 => BackendError::WeightsNotFound(msg),
        // 2 = inference error, 5 = a kernel's bounded wait ran out
        _ => BackendError::Inference(msg),
    }
}

pub struct B200Backend {
    handle: *mut TeiB200,
    output_dim: usize,
    hidden_size: usize,
    num_classes: usize,
}

// The handle is owned by the single backend thread (backends/src/lib.rs:612-647).
unsafe impl Send for B200Backend {}
// Shared by the backend threads of a multi-replica router: the `_on` entry points may be
// called concurrently with different replica indices (the library serialises equal ones).
unsafe impl Sync for B200Backend {}

impl B200Backend {
    /// Same shape as `CandleBackend::new`.  `TEI_B200_DEVICES` (comma-separated CUDA indices)
    /// selects the replicas; the default is device 0.
    pub fn new(
        model_path: &Path,
        dtype: String,
        model_type: ModelType,
        dense_paths: Option<Vec<String>>,
    ) -> Result<Self, BackendError> {
        let (mt, pool) = match model_type {
            ModelType::Classifier => (0, 0),
            ModelType::Embedding(pool) => (
                1,
                match pool {
                    Pool::Cls => 0,
                    Pool::Mean => 1,
                    Pool::Splade => 2,
                    Pool::LastToken => 3,
                },
            ),
        };
        let devices: Vec<c_int> = std::env::var("TEI_B200_DEVICES")
            .ok()
            .map(|v| v.split(',').filter_map(|s| s.trim().parse().ok()).collect())
            .unwrap_or_else(|| vec![0]);
        let dir = CString::new(model_path.to_string_lossy().as_bytes())
            .map_err(|e| BackendError::Start(e.to_string()))?;
        let dt = CString::new(dtype).map_err(|e| BackendError::Start(e.to_string()))?;
        let mut handle: *mut TeiB200 = std::ptr::null_mut();
        let mut err = vec![0 as c_char; ERR_CAP];
        let rc = unsafe {
            tei_b200_create(
                dir.as_ptr(),
                dt.as_ptr(),
                mt,
                pool,
                devices.as_ptr(),
                devices.len() as c_int,
                &mut handle,
                err.as_mut_ptr(),
                ERR_CAP,
            )
        };
        if rc != 0 {
            return Err(to_error(rc, &err));
        }
        // Dense modules run on the pooled rows inside the library, in this order.
        for dense_path in dense_paths.unwrap_or_default() {
            let path = CString::new(dense_path.as_bytes())
                .map_err(|e| BackendError::Start(e.to_string()))?;
            let mut err = vec![0 as c_char; ERR_CAP];
            let rc =
                unsafe { tei_b200_add_dense(handle, path.as_ptr(), err.as_mut_ptr(), ERR_CAP) };
            if rc != 0 {
                unsafe { tei_b200_destroy(handle) };
                return Err(to_error(rc, &err));
            }
            if err[0] != 0 {
                tracing::warn!("{}", unsafe { CStr::from_ptr(err.as_ptr()) }.to_string_lossy());
            } else {
                tracing::info!("Loaded Dense module from path: {dense_path}");
            }
        }
        let (output_dim, hidden_size, num_classes) = unsafe {
            (
                tei_b200_output_dim(handle) as usize,
                tei_b200_hidden_size(handle) as usize,
                tei_b200_num_classes(handle) as usize,
            )
        };
        Ok(Self {
            handle,
            output_dim,
            hidden_size,
            num_classes,
        })
    }
}

impl Drop for B200Backend {
    fn drop(&mut self) {
        unsafe { tei_b200_destroy(self.handle) }
    }
}

impl Backend for B200Backend {
    fn health(&self) -> Result<(), BackendError> {
        match unsafe { tei_b200_health(self.handle) } {
            0 => Ok(()),
            _ => Err(BackendError::Unhealthy),
        }
    }

    fn max_batch_size(&self) -> Option<usize> {
        match unsafe { tei_b200_max_batch_size(self.handle) } {
            n if n < 0 => None,
            n => Some(n as usize),
        }
    }

    fn is_padded(&self) -> bool {
        unsafe { tei_b200_is_padded(self.handle) != 0 }
    }

    fn embed(&self, batch: Batch) -> Result<Embeddings, BackendError> {
        self.embed_impl(None, batch)
    }

    fn predict(&self, batch: Batch) -> Result<Predictions, BackendError> {
        self.predict_impl(None, batch)
    }
}

impl B200Backend {
    /// Replicas of the handle = backend threads a router may run over it.
    pub fn num_replicas(&self) -> usize {
        unsafe { tei_b200_num_replicas(self.handle) }.max(1) as usize
    }

    /// `embed` with the whole batch on one replica; callers with different indices may overlap.
    pub fn embed_on(&self, replica: usize, batch: Batch) -> Result<Embeddings, BackendError> {
        self.embed_impl(Some(replica), batch)
    }

    /// `predict` with the whole batch on one replica.
    pub fn predict_on(&self, replica: usize, batch: Batch) -> Result<Predictions, BackendError> {
        self.predict_impl(Some(replica), batch)
    }

    fn embed_impl(&self, replica: Option<usize>, batch: Batch) -> Result<Embeddings, BackendError> {
        let batch_size = batch.len();
        let lengths: Vec<usize> = (0..batch_size)
            .map(|i| {
                (batch.cumulative_seq_lengths[i + 1] - batch.cumulative_seq_lengths[i]) as usize
            })
            .collect();
        let raw_rows: usize = batch
            .raw_indices
            .iter()
            .map(|&i| lengths.get(i as usize).copied().unwrap_or(0))
            .sum();
        let mut pooled = vec![0f32; batch.pooled_indices.len() * self.output_dim];
        let mut raw = vec![0f32; raw_rows * self.hidden_size];
        let mut err = vec![0 as c_char; ERR_CAP];
        // normalize = 0: the router normalises on the host (core/src/infer.rs:288-303)
        let rc = unsafe {
            match replica {
                None => tei_b200_embed(
                    self.handle,
                    batch.input_ids.as_ptr(),
                    batch.token_type_ids.as_ptr(),
                    batch.position_ids.as_ptr(),
                    batch.input_ids.len(),
                    batch.cumulative_seq_lengths.as_ptr(),
                    batch_size,
                    batch.max_length,
                    batch.pooled_indices.as_ptr(),
                    batch.pooled_indices.len(),
                    batch.raw_indices.as_ptr(),
                    batch.raw_indices.len(),
                    0,
                    pooled.as_mut_ptr(),
                    raw.as_mut_ptr(),
                    err.as_mut_ptr(),
                    ERR_CAP,
                ),
                Some(r) => tei_b200_embed_on(
                    self.handle,
                    r as c_int,
                    batch.input_ids.as_ptr(),
                    batch.token_type_ids.as_ptr(),
                    batch.position_ids.as_ptr(),
                    batch.input_ids.len(),
                    batch.cumulative_seq_lengths.as_ptr(),
                    batch_size,
                    batch.max_length,
                    batch.pooled_indices.as_ptr(),
                    batch.pooled_indices.len(),
                    batch.raw_indices.as_ptr(),
                    batch.raw_indices.len(),
                    0,
                    pooled.as_mut_ptr(),
                    raw.as_mut_ptr(),
                    err.as_mut_ptr(),
                    ERR_CAP,
                ),
            }
        };
        if rc != 0 {
            return Err(to_error(rc, &err));
        }
        // Same assembly as backends/candle/src/lib.rs:694-706.
        let mut embeddings =
            HashMap::with_capacity_and_hasher(batch_size, BuildNoHashHasher::default());
        for (row, i) in batch.pooled_indices.iter().enumerate() {
            let e = pooled[row * self.output_dim..(row + 1) * self.output_dim].to_vec();
            embeddings.insert(*i as usize, Embedding::Pooled(e));
        }
        let mut cumulative_length = 0;
        for i in batch.raw_indices.iter() {
            let length = lengths[*i as usize];
            let e: Vec<Vec<f32>> = (cumulative_length..cumulative_length + length)
                .map(|r| raw[r * self.hidden_size..(r + 1) * self.hidden_size].to_vec())
                .collect();
            embeddings.insert(*i as usize, Embedding::All(e));
            cumulative_length += length;
        }
        Ok(embeddings)
    }

    fn predict_impl(&self, replica: Option<usize>, batch: Batch) -> Result<Predictions, BackendError> {
        let batch_size = batch.len();
        let mut scores = vec![0f32; batch_size * self.num_classes.max(1)];
        let mut err = vec![0 as c_char; ERR_CAP];
        let rc = unsafe {
            match replica {
                None => tei_b200_predict(
                    self.handle,
                    batch.input_ids.as_ptr(),
                    batch.token_type_ids.as_ptr(),
                    batch.position_ids.as_ptr(),
                    batch.input_ids.len(),
                    batch.cumulative_seq_lengths.as_ptr(),
                    batch_size,
                    batch.max_length,
                    scores.as_mut_ptr(),
                    err.as_mut_ptr(),
                    ERR_CAP,
                ),
                Some(r) => tei_b200_predict_on(
                    self.handle,
                    r as c_int,
                    batch.input_ids.as_ptr(),
                    batch.token_type_ids.as_ptr(),
                    batch.position_ids.as_ptr(),
                    batch.input_ids.len(),
                    batch.cumulative_seq_lengths.as_ptr(),
                    batch_size,
                    batch.max_length,
                    scores.as_mut_ptr(),
                    err.as_mut_ptr(),
                    ERR_CAP,
                ),
            }
        };
        if rc != 0 {
            return Err(to_error(rc, &err));
        }
        // Same assembly as backends/candle/src/lib.rs:718-722.
        let mut predictions =
            HashMap::with_capacity_and_hasher(batch_size, BuildNoHashHasher::default());
        for i in 0..batch_size {
            predictions.insert(
                i,
                scores[i * self.num_classes..(i + 1) * self.num_classes].to_vec(),
            );
        }
        Ok(predictions)
    }
}
