//! How the ops of `paged_kv.rs` get into a model: one pre-translate rewrite rule and three arms of
//! `CudaTransform::translate_node`.  Drop into `cuda/src/rewrite_rules/paged_kv.rs`; the registered transform names
//! (`transformers/src/lib.rs:8-29`) stay as they are, and `tract::runtime_for_name("cuda").prepare(model)` picks the ops
//! up unchanged.
use crate::b200kv_sys::*;
use crate::ops::paged_kv::{CudaPagedKvCache, CudaPagedKvSdpa, CudaPagedSdpa};
use tract_core::internal::*;
use tract_transformers::ops::dyn_kv_cache::DynKeyValueCache;
use tract_transformers::ops::quant_dyn_kv_cache::QuantizedDynKeyValueCache;
use tract_transformers::ops::sdpa::Sdpa;

/// Longest sequence a cache is sized for when the model does not say (`TRACT_B200KV_MAX_TOKENS` overrides), and the
/// sequences one node may hold at once: the running state plus its frozen copies.
fn capacity() -> (i64, i32) {
    let tokens = std::env::var("TRACT_B200KV_MAX_TOKENS").ok().and_then(|s| s.parse().ok()).unwrap_or(131072);
    let seqs = std::env::var("TRACT_B200KV_MAX_SEQS").ok().and_then(|s| s.parse().ok()).unwrap_or(4);
    (tokens, seqs)
}

/// The storage format a cache node asks for: its own element type for a plain `DynKeyValueCache`, the reference's
/// own storage quantisation for a `QuantizedDynKeyValueCache` (`quantize_kv_storage[_int4]`), or, when
/// `TRACT_B200KV_BLOCK_QUANT` = `q8_1` / `q4_0` is set, the block-32 formats of tract-linalg on a plain cache.
fn storage_format(dt: DatumType, quant_bits: Option<u32>) -> TractResult<i32> {
    if let Some(bits) = quant_bits {
        return match bits {
            8 => Ok(B200KV_FMT_KIVI8),
            4 => Ok(B200KV_FMT_KIVI4),
            other => bail!("QuantizedDynKeyValueCache with {other} bits has no device form"),
        };
    }
    match std::env::var("TRACT_B200KV_BLOCK_QUANT").as_deref() {
        Ok("q8_1") => return Ok(B200KV_FMT_Q8_1),
        Ok("q4_0") => return Ok(B200KV_FMT_Q4_0),
        _ => {}
    }
    match dt {
        DatumType::F32 => Ok(B200KV_FMT_F32),
        DatumType::F16 => Ok(B200KV_FMT_F16),
        other => bail!("no paged cache for {other:?}"),
    }
}

/// What the rule needs to know about one cache node feeding an Sdpa.
struct CacheSite {
    node: usize,
    name: String,
    axis: usize,
    quant_bits: Option<u32>,
    past: TypedFact,
    input: TypedFact,
    new_tokens: OutletId,
}

fn cache_site(model: &TypedModel, outlet: OutletId) -> Option<CacheSite> {
    let n = model.node(outlet.node);
    // the cache must feed only this Sdpa, else removing it would drop a live value
    if n.outputs[outlet.slot].successors.len() != 1 {
        return None;
    }
    if let Some(c) = n.op_as::<DynKeyValueCache>() {
        return Some(CacheSite { node: n.id, name: c.name.clone(), axis: c.axis, quant_bits: None, past: c.past_sequence_fact.clone(),
                                input: c.input_sequence_fact.clone(), new_tokens: n.inputs[0] });
    }
    if let Some(c) = n.op_as::<QuantizedDynKeyValueCache>() {
        return Some(CacheSite { node: n.id, name: c.name.clone(), axis: c.axis, quant_bits: Some(c.bits), past: c.past_sequence_fact.clone(),
                                input: c.input_sequence_fact.clone(), new_tokens: n.inputs[0] });
    }
    None
}

/// Pre-translate rule (runs on the typed model, after `fuse_kv_cache_broadcast_rule` has stripped the GQA
/// unsqueeze / broadcast / reshape chain, so the caches feed the Sdpa directly): fuses
/// `{cache(K), cache(V), Sdpa(Q, K, V)}` -- both caches single-consumer, on the same axis, of the same kind -- into one
/// `CudaPagedKvSdpa` taking `[Q, K_new, V_new]`.  The pattern is that of `fuse_inplace_kv_sdpa_rule`
/// (transformers/src/ops/inplace_kv_cache.rs:293-333); unlike that rule this one keeps the caches' state contract
/// (initialisers, `resolve_symbols`, `save_to`) alive inside the fused op.
pub fn fuse_paged_kv_sdpa_rule(
    _ctx: &(),
    model: &TypedModel,
    node: &TypedNode,
    node_name: &str,
    op: &Sdpa,
) -> TractResult<Option<TypedModelPatch>> {
    if node.inputs.len() != 3 {
        return Ok(None); // an explicit mask input: stays a lone Sdpa (CudaPagedSdpa)
    }
    let (Some(k), Some(v)) = (cache_site(model, node.inputs[1]), cache_site(model, node.inputs[2])) else {
        return Ok(None);
    };
    if k.axis != v.axis || k.axis != 2 || k.quant_bits != v.quant_bits || k.node == v.node {
        return Ok(None);
    }
    let dt = k.input.datum_type;
    if v.input.datum_type != dt || !matches!(dt, DatumType::F32 | DatumType::F16) {
        return Ok(None);
    }
    // rank 4 [B, H, S, D] with batch 1 (one tract State is one sequence) and a head_dim the kernels have
    let shape = &k.input.shape;
    if shape.rank() != 4 || shape[0] != 1.to_dim() || !matches!(shape[3].to_usize(), Ok(64) | Ok(128)) {
        return Ok(None);
    }
    let Ok(format) = storage_format(dt, k.quant_bits) else { return Ok(None) };
    let scale = op.scale.as_ref().map(|t| t.cast_to_scalar::<f32>()).transpose()?;
    let (max_seq_tokens, max_seqs) = capacity();

    let mut patch = TypedModelPatch::default();
    let taps = patch.taps(model, &[node.inputs[0], k.new_tokens, v.new_tokens])?;
    let fused = patch.wire_node(
        format!("{node_name}.paged_kv_sdpa"),
        CudaPagedKvSdpa {
            name: k.name.clone(),
            axis: k.axis,
            format,
            scale: scale.map(|s| ordered_float::NotNan::new(s)).transpose()?,
            is_causal: op.is_causal,
            past_sequence_fact: k.past.clone(),
            input_sequence_fact: k.input.clone(),
            max_seq_tokens,
            max_seqs,
        },
        &taps,
    )?;
    patch.shunt_outside(model, node.id.into(), fused[0])?;
    Ok(Some(patch))
}

/// Installs the rule: called at the top of `CudaTransform::transform` (cuda/src/transform.rs), before translation.
pub fn fuse_paged_kv(model: &mut TypedModel) -> TractResult<()> {
    use tract_transformers::rewriter::Rewriter;
    Rewriter::default()
        .with_rule_for("fuse-kv-broadcast", tract_transformers::ops::sdpa::fuse_kv_cache_broadcast_rule)
        .with_rule_for("fuse-paged-kv-sdpa", fuse_paged_kv_sdpa_rule)
        .rewrite(&(), model)
}

/// The arms of `CudaTransform::translate_node` (cuda/src/transform.rs:411-527), placed BEFORE `try_make_cuda_op`
/// (:502) and in place of the `Sdpa` arm that calls `convert_sdpa_to_cuda_flash_attn` (:431-437).  Returns the op to
/// wire for `node`, or None when the node is none of ours.
pub fn translate_paged(source: &TypedModel, node: &TypedNode) -> TractResult<Option<Box<dyn TypedOp>>> {
    let (max_seq_tokens, max_seqs) = capacity();
    // (i) the fused op is already a device op: wired as it is, its inputs synced to the device
    if let Some(op) = node.op_as::<CudaPagedKvSdpa>() {
        return Ok(Some(Box::new(op.clone())));
    }
    // (ii) a lone cache (its consumer was not an Sdpa): in-place append, contiguous view out
    if let Some(op) = node.op_as::<DynKeyValueCache>() {
        let dt = op.input_sequence_fact.datum_type;
        if op.axis == 2 && op.input_sequence_fact.rank() == 4 {
            if let Ok(format) = storage_format(dt, None) {
                return Ok(Some(Box::new(CudaPagedKvCache {
                    name: op.name.clone(), axis: op.axis, format, per_token: false,
                    past_sequence_fact: op.past_sequence_fact.clone(), input_sequence_fact: op.input_sequence_fact.clone(),
                    max_seq_tokens, max_seqs,
                })));
            }
        }
        return Ok(None); // falls through to GpuDynKVCache
    }
    if let Some(op) = node.op_as::<QuantizedDynKeyValueCache>() {
        if op.axis == 2 && op.input_sequence_fact.rank() == 4 {
            if let Ok(format) = storage_format(op.input_sequence_fact.datum_type, Some(op.bits)) {
                return Ok(Some(Box::new(CudaPagedKvCache {
                    name: op.name.clone(), axis: op.axis, format, per_token: !op.per_channel,
                    past_sequence_fact: op.past_sequence_fact.clone(), input_sequence_fact: op.input_sequence_fact.clone(),
                    max_seq_tokens, max_seqs,
                })));
            }
        }
        return Ok(None); // stays on the CPU, as today
    }
    // (iii) a lone Sdpa: any head_dim <= 256, f32 or f16, optional mask -- no cast / pad / reshape wiring around it
    if let Some(op) = node.op_as::<Sdpa>() {
        let facts = source.node_input_facts(node.id)?;
        let dt = facts[0].datum_type;
        let d_ok = facts[0].shape.last().and_then(|d| d.to_usize().ok()).map(|d| d <= 256).unwrap_or(false);
        if matches!(dt, DatumType::F32 | DatumType::F16) && facts.iter().take(3).all(|f| f.datum_type == dt) && d_ok {
            let scale = op.scale.as_ref().map(|t| t.cast_to_scalar::<f32>()).transpose()?;
            return Ok(Some(Box::new(CudaPagedSdpa {
                scale: scale.map(|s| ordered_float::NotNan::new(s)).transpose()?,
                is_causal: op.is_causal,
            })));
        }
    }
    Ok(None)
}

// In `translate_node`, right after `let input_facts = source.node_input_facts(node.id)?;`:
//
//     #[cfg(feature = "b200kv")]
//     if let Some(gpu_op) = crate::rewrite_rules::paged_kv::translate_paged(source, node)? {
//         let device_inputs = sync_inputs_if_required(target, node, mapping, DeviceSyncKind::ToDevice)?;
//         let outlet_ids = target.wire_node(node.name.clone(), gpu_op, &device_inputs)?;
//         return sync_model_outputs_if_required(source, node, target, outlet_ids);
//     }
//
// and in `CudaTransform::transform`, before the translation pass:
//
//     #[cfg(feature = "b200kv")]
//     crate::rewrite_rules::paged_kv::fuse_paged_kv(model)?;
