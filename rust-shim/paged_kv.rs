//! The ops tract-cuda wires in place of `GpuDynKVCache` / `CudaFlashAttention` when the `b200kv` feature is on.
//! Drop into `cuda/src/ops/paged_kv.rs`.
//!
//!  * `CudaPagedKvSdpa`   stateful, inputs `[Q, K_new, V_new]`: the fused `{cache(K), cache(V), Sdpa}` subgraph (the CPU
//!                        form of it is `InPlaceKvSdpa`, transformers/src/ops/inplace_kv_cache.rs:135-216)
//!  * `CudaPagedKvCache`  stateful, input `[X_new]`: a lone `DynKeyValueCache` / `QuantizedDynKeyValueCache` whose
//!                        consumer is not an Sdpa; appends in place and hands a contiguous view out
//!  * `CudaPagedSdpa`     stateless, inputs `[Q, K, V]` or `[Q, K, V, mask]`: a lone `Sdpa`
//!
//! One library handle holds the pages of one op node; each tract `State` (one running sequence) owns one sequence
//! id in it.  `freeze` forks the sequence on the device (no host round trip, unlike
//! gpu/src/ops/dyn_kv_cache.rs:116-125), `unfreeze` forks the frozen copy again, so a frozen state can be thawed any
//! number of times.
use crate::b200kv_sys::*;
use crate::context::with_cuda_stream;
use std::os::raw::c_void;
use std::sync::{Arc, Mutex};
use tract_core::internal::*;
use tract_core::ops::OpStateFreeze;
use tract_gpu::fact::DeviceTypedFactExt;
use tract_gpu::session_handler::make_tensor_for_node;
use tract_gpu::tensor::{DeviceTensor, DeviceTensorExt, IntoDevice};
use tract_transformers::ops::dyn_kv_cache::DynKeyValueCacheState;

// ------------------------------------------------------------------------------------------------
// helpers
// ------------------------------------------------------------------------------------------------

fn dtype_code(dt: DatumType) -> TractResult<i32> {
    match dt {
        DatumType::F32 => Ok(B200KV_F32),
        DatumType::F16 => Ok(B200KV_F16),
        other => bail!("b200kv: unsupported datum type {other:?} (f32 and f16 are tract's device float types)"),
    }
}

/// Raw device address of element 0 and the strides in elements (gpu/src/tensor/mod.rs:113-146).
fn raw_parts(t: &DeviceTensor) -> (*const c_void, TVec<i64>) {
    let addr = t.device_buffer_ptr() as usize + t.buffer_offset::<usize>();
    (addr as *const c_void, t.strides().iter().map(|s| *s as i64).collect())
}

fn raw_stream(stream: &crate::context::TractCudaStream) -> *mut c_void {
    stream.cu_stream() as *mut c_void
}

/// Owner of one `b200kv_cache*`.  The library wants one thread at a time per handle (like an `OpState`); states that
/// share a handle (frozen copies, sibling sequences of one plan) go through the mutex.
pub struct PagedCache {
    raw: *mut b200kv_cache,
    pub cfg: b200kv_config,
}
unsafe impl Send for PagedCache {}
unsafe impl Sync for PagedCache {}

impl PagedCache {
    pub fn new(cfg: b200kv_config) -> TractResult<Self> {
        let mut raw = std::ptr::null_mut();
        ck(unsafe { b200kv_create(&cfg, &mut raw) })?;
        Ok(PagedCache { raw, cfg })
    }
}
impl Drop for PagedCache {
    fn drop(&mut self) {
        unsafe { b200kv_destroy(self.raw) };
    }
}
impl std::fmt::Debug for PagedCache {
    fn fmt(&self, f: &mut std::fmt::Formatter) -> std::fmt::Result {
        write!(f, "PagedCache(format={}, Hkv={}, D={})", self.cfg.format, self.cfg.n_kv_heads, self.cfg.head_dim)
    }
}

/// One sequence of a shared handle; freed when the last owner goes.
#[derive(Debug)]
pub struct PagedSeq {
    cache: Arc<Mutex<PagedCache>>,
    id: i32,
}
impl PagedSeq {
    fn new(cache: Arc<Mutex<PagedCache>>) -> TractResult<Self> {
        let mut id = -1;
        ck(unsafe { b200kv_seq_new(cache.lock().unwrap().raw, &mut id) })?;
        Ok(PagedSeq { cache, id })
    }
    fn len(&self) -> TractResult<usize> {
        let n = unsafe { b200kv_seq_len(self.cache.lock().unwrap().raw, self.id) };
        ensure!(n >= 0, "b200kv: sequence {} is not live", self.id);
        Ok(n as usize)
    }
    /// A device-side copy of this sequence under a new id of the same handle.
    fn fork(&self) -> TractResult<PagedSeq> {
        let mut id = -1;
        with_cuda_stream(|s| ck(unsafe { b200kv_fork(self.cache.lock().unwrap().raw, self.id, &mut id, raw_stream(s)) }))?;
        Ok(PagedSeq { cache: self.cache.clone(), id })
    }
}
impl Drop for PagedSeq {
    fn drop(&mut self) {
        if let Ok(c) = self.cache.lock() {
            unsafe { b200kv_seq_free(c.raw, self.id) };
        }
    }
}

// ------------------------------------------------------------------------------------------------
// CudaPagedKvSdpa: {DynKeyValueCache(K), DynKeyValueCache(V), Sdpa(Q, K, V)} as one stateful op
// ------------------------------------------------------------------------------------------------

#[derive(Clone, Debug, PartialEq, Eq, Hash)]
pub struct CudaPagedKvSdpa {
    /// name of the K cache node: the state initialiser keeps it (`init_tensor_fact`)
    pub name: String,
    pub axis: usize,
    /// `B200KV_FMT_*`: the input's own type for a plain `DynKeyValueCache`, KIVI8 / KIVI4 for a
    /// `QuantizedDynKeyValueCache`, Q8_1 / Q4_0 when the `b200kv_block_quant_kv` transform asked for them
    pub format: i32,
    pub scale: Option<ordered_float::NotNan<f32>>,
    pub is_causal: bool,
    pub past_sequence_fact: TypedFact,
    pub input_sequence_fact: TypedFact,
    /// longest sequence the page table is sized for, and sequences that may be live at once (frozen copies included)
    pub max_seq_tokens: i64,
    pub max_seqs: i32,
}

impl Op for CudaPagedKvSdpa {
    fn name(&self) -> StaticName {
        "CudaPagedKvSdpa".into()
    }
    fn info(&self) -> TractResult<Vec<String>> {
        Ok(vec![format!("axis={}, format={}, causal={}, scale={:?}", self.axis, self.format, self.is_causal, self.scale)])
    }
    op_as_typed_op!();
}

impl EvalOp for CudaPagedKvSdpa {
    fn is_stateless(&self) -> bool {
        false
    }
    fn state(&self, _session: &TurnState, node_id: usize) -> TractResult<Option<Box<dyn OpState>>> {
        Ok(Some(Box::new(CudaPagedKvSdpaState { node_id, op: self.clone(), seq: None })))
    }
}

impl TypedOp for CudaPagedKvSdpa {
    fn output_facts(&self, inputs: &[&TypedFact]) -> TractResult<TVec<TypedFact>> {
        ensure!(inputs.len() == 3, "CudaPagedKvSdpa expects [Q, K_new, V_new]");
        // the attention output has Q's shape and type, on the device
        tract_gpu::utils::facts_to_device_facts(inputs, |facts| Ok(tvec!(facts[0].without_value())))
            .with_context(|| format!("Error while computing facts for {:?}", self.name()))
    }
    as_op!();
}

#[derive(Debug)]
pub struct CudaPagedKvSdpaState {
    node_id: usize,
    op: CudaPagedKvSdpa,
    /// created at the first `eval` / `load_from`, when the kv-head count and head_dim are known
    seq: Option<PagedSeq>,
}

impl CudaPagedKvSdpaState {
    fn ensure_seq(&mut self, n_kv_heads: usize, head_dim: usize, n_q_heads: usize) -> TractResult<&PagedSeq> {
        if self.seq.is_none() {
            let cfg = b200kv_config {
                device: 0, // tract-cuda pins device 0 (cuda/src/context.rs:65)
                format: self.op.format,
                n_kv_heads: n_kv_heads as i32,
                head_dim: head_dim as i32,
                has_values: 1,
                max_seqs: self.op.max_seqs,
                max_seq_tokens: self.op.max_seq_tokens,
                pool_tokens: self.op.max_seq_tokens * self.op.max_seqs as i64,
                flags: 0,
                max_q_heads: n_q_heads as i32,
            };
            let cache = Arc::new(Mutex::new(PagedCache::new(cfg)?));
            self.seq = Some(PagedSeq::new(cache)?);
        }
        Ok(self.seq.as_ref().unwrap())
    }

    /// Appends `[1, Hkv, S, D]` K and V tensors (device or host values) to the sequence.
    fn append(&mut self, k: &TValue, v: &TValue, n_q_heads: usize) -> TractResult<()> {
        let (kd, vd) = (k.to_device_tensor()?, v.to_device_tensor()?);
        ensure!(kd.rank() == 4 && kd.shape() == vd.shape() && kd.shape()[0] == 1, "paged KV cache: K / V must be [1, Hkv, S, D]");
        ensure!(self.op.axis == 2, "paged KV cache: the sequence axis must be 2 ([B, H, S, D])");
        let (hkv, s, d) = (kd.shape()[1], kd.shape()[2], kd.shape()[3]);
        let dt = dtype_code(kd.datum_type())?;
        let seq = self.ensure_seq(hkv, d, n_q_heads)?;
        let ((kp, ks), (vp, vs)) = (raw_parts(kd), raw_parts(vd));
        with_cuda_stream(|stream| {
            ck(unsafe {
                b200kv_append(seq.cache.lock().unwrap().raw, 1, &seq.id, s as i32, kp, ks.as_ptr(), vp, vs.as_ptr(), dt, raw_stream(stream))
            })
        })
    }

    /// Drops the tail of the sequence (speculative-decoding rollback): the inherent `truncate` of
    /// `DynKeyValueCacheState` (transformers/src/ops/dyn_kv_cache.rs:112-119) without the host round trip of
    /// gpu/src/ops/dyn_kv_cache.rs:116-125.
    pub fn truncate(&mut self, len: usize) -> TractResult<()> {
        match &self.seq {
            Some(seq) => ck(unsafe { b200kv_truncate(seq.cache.lock().unwrap().raw, seq.id, len as i64) }),
            None => bail!("Can not truncate a zero-len kv-cache value"),
        }
    }
}

impl OpState for CudaPagedKvSdpaState {
    fn init_tensor_fact(&self) -> Option<(String, TypedFact)> {
        Some((self.op.name.clone(), self.op.past_sequence_fact.clone()))
    }

    // must be true, or the past-length symbol never resolves (core/src/plan.rs:282-292)
    fn has_init_tensor_fact(&self) -> bool {
        true
    }

    fn resolve_symbols(&mut self, state: &mut TurnState) -> TractResult<()> {
        // the cached tensor no longer exists as a tensor: the library knows the length
        let mut shape: TVec<usize> = self.op.past_sequence_fact.shape.iter().map(|d| d.to_usize().unwrap_or(0)).collect();
        let concrete = match &self.seq {
            Some(seq) => {
                shape[self.op.axis] = seq.len()?;
                Some(&*shape)
            }
            None => None,
        };
        DynKeyValueCacheState::resolve_symbols(state, self.op.past_sequence_fact.clone(), concrete)
    }

    /// Initial K then V tensors: appended to the empty sequence.  A quantised format re-quantises them token by token,
    /// as `QuantizedDynKvCacheState::load_from` does (transformers/src/ops/quant_dyn_kv_cache.rs:462-472).
    fn load_from(&mut self, state: &mut TurnState, states: &mut dyn Iterator<Item = TValue>) -> TractResult<()> {
        let k = states.next().context("Not enough state initializers")?;
        let v = states.next().context("CudaPagedKvSdpa load_from: expected V state after K")?;
        DynKeyValueCacheState::resolve_symbols(state, self.op.past_sequence_fact.clone(), Some(k.shape()))?;
        self.seq = None; // a fresh sequence: whatever was cached is dropped
        if k.shape()[self.op.axis] > 0 {
            let (kd, vd) = (k.into_tensor().into_device()?.into_tensor().into_tvalue(), v.into_tensor().into_device()?.into_tensor().into_tvalue());
            let hq = kd.shape()[1]; // the group size is not known yet: sized for it at the first eval if larger
            self.append(&kd, &vd, hq)?;
        }
        Ok(())
    }

    /// `[K, V]` as `[1, Hkv, len, D]` host tensors of the model's type (dequantised for a quantised format: what the
    /// unfused cache op would have returned, quant_dyn_kv_cache.rs:493).
    fn save_to(&self, states: &mut Vec<TValue>) -> TractResult<()> {
        let Some(seq) = &self.seq else { bail!("KV cache {} was never initialized", self.op.name) };
        let (cfg, len) = (seq.cache.lock().unwrap().cfg, seq.len()?);
        let dt = self.op.input_sequence_fact.datum_type;
        let shape = [1, cfg.n_kv_heads as usize, len, cfg.head_dim as usize];
        let (k, v) = (DeviceTensor::uninitialized_dt(dt, &shape)?, DeviceTensor::uninitialized_dt(dt, &shape)?);
        let st = [(len * cfg.head_dim as usize) as i64, cfg.head_dim as i64];
        with_cuda_stream(|stream| {
            ck(unsafe {
                b200kv_export(seq.cache.lock().unwrap().raw, seq.id, raw_parts(&k).0 as *mut c_void, st.as_ptr(),
                              raw_parts(&v).0 as *mut c_void, st.as_ptr(), dtype_code(dt)?, raw_stream(stream))
            })
        })?;
        states.push(k.to_host()?.into_tensor().into_tvalue());
        states.push(v.to_host()?.into_tensor().into_tvalue());
        Ok(())
    }

    fn eval(&mut self, session: &mut TurnState, _op: &dyn Op, inputs: TVec<TValue>) -> TractResult<TVec<TValue>> {
        ensure!(inputs.len() == 3, "CudaPagedKvSdpa expects [Q, K_new, V_new]");
        let q = inputs[0].to_device_tensor()?;
        ensure!(q.rank() == 4 && q.shape()[0] == 1, "CudaPagedKvSdpa: Q must be [1, Hq, S, D]");
        let (hq, s) = (q.shape()[1], q.shape()[2]);
        self.append(&inputs[1], &inputs[2], hq)?;
        let out = make_tensor_for_node(session, self.node_id, q.datum_type(), q.shape())?; // arena view or owned
        let seq = self.seq.as_ref().unwrap();
        let ((qp, qs), (op, os)) = (raw_parts(q), raw_parts(&out));
        let scale = self.op.scale.map(|s| s.into_inner()).unwrap_or(0.0); // <= 0 selects 1 / sqrt(D)
        with_cuda_stream(|stream| {
            ck(unsafe {
                b200kv_attend(seq.cache.lock().unwrap().raw, 1, &seq.id, hq as i32, s as i32, qp, qs.as_ptr(), op as *mut c_void,
                              os.as_ptr(), dtype_code(q.datum_type())?, scale, self.op.is_causal as i32, raw_stream(stream))
            })
        })?;
        Ok(tvec!(out.into_tensor().into_tvalue()))
    }
}

#[derive(Debug)]
pub struct FrozenCudaPagedKvSdpaState {
    node_id: usize,
    op: CudaPagedKvSdpa,
    seq: Option<Arc<PagedSeq>>,
}

impl OpStateFreeze for CudaPagedKvSdpaState {
    /// The running state goes on: the frozen copy is a device-side fork of the sequence.
    fn freeze(&self) -> Box<dyn FrozenOpState + 'static> {
        let seq = self.seq.as_ref().map(|s| Arc::new(s.fork().expect("b200kv_fork failed")));
        Box::new(FrozenCudaPagedKvSdpaState { node_id: self.node_id, op: self.op.clone(), seq })
    }
    /// The running state ends here: its sequence moves into the frozen state as it is.
    fn freeze_into(self: Box<Self>) -> Box<dyn FrozenOpState> {
        Box::new(FrozenCudaPagedKvSdpaState { node_id: self.node_id, op: self.op, seq: self.seq.map(Arc::new) })
    }
}

impl FrozenOpState for FrozenCudaPagedKvSdpaState {
    fn unfreeze(&self) -> Box<dyn OpState> {
        let seq = self.seq.as_ref().map(|s| s.fork().expect("b200kv_fork failed"));
        Box::new(CudaPagedKvSdpaState { node_id: self.node_id, op: self.op.clone(), seq })
    }
}

// ------------------------------------------------------------------------------------------------
// CudaPagedKvCache: a lone cache node (its consumer is not an Sdpa)
// ------------------------------------------------------------------------------------------------

#[derive(Clone, Debug, PartialEq, Eq, Hash)]
pub struct CudaPagedKvCache {
    pub name: String,
    pub axis: usize,
    pub format: i32,
    /// a lone KIVI cache: per token (the Value layout) instead of per channel
    pub per_token: bool,
    pub past_sequence_fact: TypedFact,
    pub input_sequence_fact: TypedFact,
    pub max_seq_tokens: i64,
    pub max_seqs: i32,
}

impl Op for CudaPagedKvCache {
    fn name(&self) -> StaticName {
        "CudaPagedKvCache".into()
    }
    fn info(&self) -> TractResult<Vec<String>> {
        Ok(vec![format!("axis={}, format={}", self.axis, self.format)])
    }
    op_as_typed_op!();
}

impl EvalOp for CudaPagedKvCache {
    fn is_stateless(&self) -> bool {
        false
    }
    fn state(&self, _session: &TurnState, node_id: usize) -> TractResult<Option<Box<dyn OpState>>> {
        Ok(Some(Box::new(CudaPagedKvCacheState { node_id, op: self.clone(), seq: None })))
    }
}

impl TypedOp for CudaPagedKvCache {
    /// The whole cache, axis grown to P + S, owned by the state (gpu/src/ops/dyn_kv_cache.rs:241-256).
    fn output_facts(&self, inputs: &[&TypedFact]) -> TractResult<TVec<TypedFact>> {
        ensure!(inputs.len() == 1);
        let mut facts = tract_gpu::utils::facts_to_device_facts(inputs, |facts| {
            let mut fact = facts[0].without_value();
            fact.shape.set(
                self.axis,
                self.past_sequence_fact.shape.dims()[self.axis].clone() + self.input_sequence_fact.shape.dims()[self.axis].clone(),
            );
            Ok(tvec!(fact))
        })
        .with_context(|| format!("Error while computing facts for {:?}", self.name()))?;
        facts[0].as_device_fact_mut().unwrap().state_owned = true;
        Ok(facts)
    }
    as_op!();
}

#[derive(Debug)]
pub struct CudaPagedKvCacheState {
    node_id: usize,
    op: CudaPagedKvCache,
    seq: Option<PagedSeq>,
}

impl CudaPagedKvCacheState {
    fn append(&mut self, x: &TValue) -> TractResult<()> {
        let xd = x.to_device_tensor()?;
        ensure!(xd.rank() == 4 && xd.shape()[0] == 1 && self.op.axis == 2, "paged KV cache: input must be [1, H, S, D], axis 2");
        let (h, s, d) = (xd.shape()[1], xd.shape()[2], xd.shape()[3]);
        if self.seq.is_none() {
            let cfg = b200kv_config {
                device: 0,
                format: self.op.format,
                n_kv_heads: h as i32,
                head_dim: d as i32,
                has_values: 0,
                max_seqs: self.op.max_seqs,
                max_seq_tokens: self.op.max_seq_tokens,
                pool_tokens: self.op.max_seq_tokens * self.op.max_seqs as i64,
                flags: self.op.per_token as i32,
                max_q_heads: 0,
            };
            self.seq = Some(PagedSeq::new(Arc::new(Mutex::new(PagedCache::new(cfg)?)))?);
        }
        let seq = self.seq.as_ref().unwrap();
        let (xp, xs) = raw_parts(xd);
        with_cuda_stream(|stream| {
            ck(unsafe {
                b200kv_append(seq.cache.lock().unwrap().raw, 1, &seq.id, s as i32, xp, xs.as_ptr(), std::ptr::null(), std::ptr::null(),
                              dtype_code(xd.datum_type())?, raw_stream(stream))
            })
        })
    }

    /// The cache as one contiguous `[1, H, len, D]` device tensor of type `dt`.
    fn materialize(&self, session: Option<&TurnState>, dt: DatumType) -> TractResult<DeviceTensor> {
        let seq = self.seq.as_ref().context("KV cache was never initialized")?;
        let (cfg, len) = (seq.cache.lock().unwrap().cfg, seq.len()?);
        let shape = [1, cfg.n_kv_heads as usize, len, cfg.head_dim as usize];
        let out = match session {
            Some(s) => make_tensor_for_node(s, self.node_id, dt, &shape)?,
            None => DeviceTensor::uninitialized_dt(dt, &shape)?,
        };
        let st = [(len * cfg.head_dim as usize) as i64, cfg.head_dim as i64];
        with_cuda_stream(|stream| {
            ck(unsafe {
                b200kv_export(seq.cache.lock().unwrap().raw, seq.id, raw_parts(&out).0 as *mut c_void, st.as_ptr(), std::ptr::null_mut(),
                              std::ptr::null(), dtype_code(dt)?, raw_stream(stream))
            })
        })?;
        Ok(out)
    }

    pub fn truncate(&mut self, len: usize) -> TractResult<()> {
        match &self.seq {
            Some(seq) => ck(unsafe { b200kv_truncate(seq.cache.lock().unwrap().raw, seq.id, len as i64) }),
            None => bail!("Can not truncate a zero-len kv-cache value"),
        }
    }
}

impl OpState for CudaPagedKvCacheState {
    fn init_tensor_fact(&self) -> Option<(String, TypedFact)> {
        Some((self.op.name.clone(), self.op.past_sequence_fact.clone()))
    }
    fn has_init_tensor_fact(&self) -> bool {
        true
    }
    fn resolve_symbols(&mut self, state: &mut TurnState) -> TractResult<()> {
        let mut shape: TVec<usize> = self.op.past_sequence_fact.shape.iter().map(|d| d.to_usize().unwrap_or(0)).collect();
        let concrete = match &self.seq {
            Some(seq) => {
                shape[self.op.axis] = seq.len()?;
                Some(&*shape)
            }
            None => None,
        };
        DynKeyValueCacheState::resolve_symbols(state, self.op.past_sequence_fact.clone(), concrete)
    }
    fn load_from(&mut self, state: &mut TurnState, states: &mut dyn Iterator<Item = TValue>) -> TractResult<()> {
        let x = states.next().context("Not enough state initializers")?;
        DynKeyValueCacheState::resolve_symbols(state, self.op.past_sequence_fact.clone(), Some(x.shape()))?;
        self.seq = None;
        if x.shape()[self.op.axis] > 0 {
            self.append(&x.into_tensor().into_device()?.into_tensor().into_tvalue())?;
        }
        Ok(())
    }
    fn save_to(&self, states: &mut Vec<TValue>) -> TractResult<()> {
        if self.seq.is_none() {
            bail!("KV cache {} was never initialized", self.op.name)
        }
        let t = self.materialize(None, self.op.input_sequence_fact.datum_type)?;
        states.push(t.to_host()?.into_tensor().into_tvalue());
        Ok(())
    }
    /// Appends in place (touches only the new tokens), then hands the consumer the contiguous tensor the op's contract
    /// promises.  Consumers that are an Sdpa never get here: the pre-translate rule fuses them into CudaPagedKvSdpa.
    fn eval(&mut self, session: &mut TurnState, _op: &dyn Op, inputs: TVec<TValue>) -> TractResult<TVec<TValue>> {
        ensure!(inputs.len() == 1);
        let dt = inputs[0].datum_type();
        self.append(&inputs[0])?;
        let out = self.materialize(Some(session), dt)?;
        Ok(tvec!(out.into_tensor().into_tvalue()))
    }
}

#[derive(Debug)]
pub struct FrozenCudaPagedKvCacheState {
    node_id: usize,
    op: CudaPagedKvCache,
    seq: Option<Arc<PagedSeq>>,
}

impl OpStateFreeze for CudaPagedKvCacheState {
    fn freeze(&self) -> Box<dyn FrozenOpState + 'static> {
        let seq = self.seq.as_ref().map(|s| Arc::new(s.fork().expect("b200kv_fork failed")));
        Box::new(FrozenCudaPagedKvCacheState { node_id: self.node_id, op: self.op.clone(), seq })
    }
    fn freeze_into(self: Box<Self>) -> Box<dyn FrozenOpState> {
        Box::new(FrozenCudaPagedKvCacheState { node_id: self.node_id, op: self.op, seq: self.seq.map(Arc::new) })
    }
}

impl FrozenOpState for FrozenCudaPagedKvCacheState {
    fn unfreeze(&self) -> Box<dyn OpState> {
        let seq = self.seq.as_ref().map(|s| s.fork().expect("b200kv_fork failed"));
        Box::new(CudaPagedKvCacheState { node_id: self.node_id, op: self.op.clone(), seq })
    }
}

// ------------------------------------------------------------------------------------------------
// CudaPagedSdpa: a lone Sdpa on dense tensors (replaces CudaFlashAttention, cuda/src/ops/flash_attn.rs:6-76)
// ------------------------------------------------------------------------------------------------

#[derive(Clone, Debug, PartialEq, Eq, Hash)]
pub struct CudaPagedSdpa {
    pub scale: Option<ordered_float::NotNan<f32>>,
    pub is_causal: bool,
}

impl Op for CudaPagedSdpa {
    fn name(&self) -> StaticName {
        "CudaPagedSdpa".into()
    }
    op_as_typed_op!();
}

impl EvalOp for CudaPagedSdpa {
    fn is_stateless(&self) -> bool {
        true
    }
    fn eval_with_session(&self, node_id: usize, session: &TurnState, inputs: TVec<TValue>) -> TractResult<TVec<TValue>> {
        ensure!(inputs.len() == 3 || inputs.len() == 4, "Sdpa expects [Q, K, V] or [Q, K, V, mask]");
        let (q, k, v) = (inputs[0].to_device_tensor()?, inputs[1].to_device_tensor()?, inputs[2].to_device_tensor()?);
        let rank = q.rank();
        ensure!((rank == 3 || rank == 4) && k.rank() == rank && v.rank() == rank, "Sdpa: rank 3 or 4");
        // rank 3 [B, S, D] is rank 4 with one head
        let dims = |t: &DeviceTensor| -> (usize, usize, usize, usize) {
            let s = t.shape();
            if rank == 4 { (s[0], s[1], s[2], s[3]) } else { (s[0], 1, s[1], s[2]) }
        };
        let strides3 = |t: &DeviceTensor| -> [i64; 3] {
            let s = t.strides();
            if rank == 4 { [s[0] as i64, s[1] as i64, s[2] as i64] } else { [s[0] as i64, 0, s[1] as i64] }
        };
        let ((b, hq, s, d), (_, hkv, t, _)) = (dims(q), dims(k));
        let out = make_tensor_for_node(session, node_id, q.datum_type(), q.shape())?;
        let (qs, ks, vs, os) = (strides3(q), strides3(k), strides3(v), strides3(&out));
        let (mask_ptr, mask_strides, mask_dt) = match inputs.get(3) {
            Some(m) => {
                let m = m.to_device_tensor()?;
                // broadcast axes (extent 1) get stride 0; a rank-3 mask has no head axis
                let (sh, st) = (m.shape(), m.strides());
                let at = |ax: usize| if sh[ax] == 1 { 0 } else { st[ax] as i64 };
                let ms = if m.rank() == 4 { [at(0), at(1), st[2] as i64, st[3] as i64] } else { [at(0), 0, st[1] as i64, st[2] as i64] };
                (raw_parts(m).0, ms, dtype_code(m.datum_type())?)
            }
            None => (std::ptr::null(), [0i64; 4], 0),
        };
        let scale = self.scale.map(|s| s.into_inner()).unwrap_or(0.0);
        with_cuda_stream(|stream| {
            ck(unsafe {
                b200kv_sdpa(raw_parts(q).0, qs.as_ptr(), raw_parts(k).0, ks.as_ptr(), raw_parts(v).0, vs.as_ptr(), mask_ptr,
                            mask_strides.as_ptr(), mask_dt, raw_parts(&out).0 as *mut c_void, os.as_ptr(), b as i32, hq as i32,
                            hkv as i32, s as i32, t as i32, d as i32, dtype_code(q.datum_type())?, scale, self.is_causal as i32,
                            raw_stream(stream))
            })
        })?;
        Ok(tvec!(out.into_tensor().into_tvalue()))
    }
}

impl TypedOp for CudaPagedSdpa {
    fn output_facts(&self, inputs: &[&TypedFact]) -> TractResult<TVec<TypedFact>> {
        tract_gpu::utils::facts_to_device_facts(inputs, |facts| Ok(tvec!(facts[0].without_value())))
            .with_context(|| format!("Error while computing facts for {:?}", self.name()))
    }
    as_op!();
}
