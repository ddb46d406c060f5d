"""Loading a layer saved by the upstream quantizer into a QuantizedLinear.

The per-layer file written by lib/algo/finetune.py:238-257 upstream holds
{trellis, SU, SV, Wscale, proxy_err, tlut, rcp, tp_rank}.  unpack_quip (lib/utils/data_utils.py:281-307)
copies it into the module and folds the weight scale into a sign vector: into SV for an unsplit layer,
per tensor-parallel chunk into SU for a row-parallel layer (rcp = 1) and into SV for a column-parallel
one (rcp = 2).  Upstream hard-codes 8 chunks there; the saved tp_rank is used here, which is the same
number for every file upstream writes.
"""
import torch


def unpack_quip(module, saved_layer):
    module.trellis.copy_(saved_layer['trellis'])
    if module.tlut is not None:
        module.tlut.copy_(saved_layer['tlut'].float().to(torch.float16))
    SU, SV = saved_layer['SU'].float(), saved_layer['SV'].float()
    Wscale = torch.as_tensor(saved_layer['Wscale']).float()
    if 'rcp' not in saved_layer:
        module.SU.copy_(SU)
        module.SV.copy_(SV * Wscale)
        return module
    rcp = int(saved_layer['rcp'])
    chunks = int(saved_layer.get('tp_rank', 8))
    module.rcp.copy_(torch.tensor(rcp))
    module.tp_rank.copy_(torch.tensor(chunks))
    if rcp == 1:
        module.SU.copy_((SU.reshape(chunks, -1) * Wscale.reshape(-1, 1)).reshape(SU.shape))
        module.SV.copy_(SV)
    elif rcp == 2:
        module.SU.copy_(SU)
        module.SV.copy_((SV.reshape(chunks, -1) * Wscale.reshape(-1, 1)).reshape(SV.shape))
    else:
        module.SU.copy_(SU)
        module.SV.copy_(SV * Wscale)
    return module


# ---------------------------------------------------------------------------------------------------------
# Whole-model ingestion: an upstream (hfized) state dict + quip_params -> QtipLlama
# ---------------------------------------------------------------------------------------------------------
_PROJ = {"q": "self_attn.q_proj", "k": "self_attn.k_proj", "v": "self_attn.v_proj", "o": "self_attn.o_proj",
         "gate": "mlp.gate_proj", "up": "mlp.up_proj", "down": "mlp.down_proj"}


def check_quip_params(quip_params, shape):
    """Refuse what the decode path does not build, with the key that is at fault.  `quip_params` is the dict the
    upstream quantizer stores in the HF config (quantize_llama/quantize_finetune_llama.py:116-129) and the model
    reads at model/llama.py:306-317, 445-452 (incl. the optional K_v_proj and skip_list)."""
    need = dict(L=16, V=2, tlut_bits=9, decode_mode="quantlut_sym", td_x=16, td_y=16)
    for key, want in need.items():
        got = quip_params.get(key)
        if got != want:
            raise ValueError(f"quip_params[{key!r}] = {got!r}: the fused decode path is built for {want!r} "
                             "(the HYB code with the 16x16 kernel layout)")
    K = int(quip_params["K"])
    if K not in (2, 3, 4):
        raise ValueError(f"quip_params['K'] = {K}: 2, 3 or 4 bits per weight")
    if int(quip_params.get("K_v_proj", K)) != K:
        raise ValueError("quip_params['K_v_proj'] differs from K: q/k/v share one launch and must use one bitrate")
    if quip_params.get("skip_list"):
        raise ValueError(f"quip_params['skip_list'] = {quip_params['skip_list']!r}: unquantized (skipped) linears are not "
                         "part of the decode path")
    if K != shape.K:
        raise ValueError(f"quip_params['K'] = {K} but the model was built for K = {shape.K}")
    return K


def load_state_dict_into(model, state_dict, quip_params, prefix="model."):
    """Copy an upstream QTIP Llama state dict into a QtipLlama (single GPU, unfused q/k/v and gate/up).

    Keys per linear (lib/linear/quantized_linear.py:41-67 upstream): `{prefix}layers.{i}.{proj}.trellis` int16
    (m/16 * n/16, 16K), `.tlut` fp16 (512, 2), `.SU` fp16 (n), `.SV` fp32 (m) with the weight scale already folded in
    by unpack_quip, `.rcp`, `.tp_rank`; per layer `input_layernorm.weight`, `post_attention_layernorm.weight`; then
    `{prefix}embed_tokens.weight`, `{prefix}norm.weight`, `lm_head.weight`.  Layers quantized with a tensor-parallel
    layout (rcp != 0) are refused: their transforms run per chunk, which this single-GPU model does not do.
    Shapes and dtypes are checked; missing keys raise KeyError naming the key."""
    assert model.tp == 1 and not model.fuse_qkv, "load into a single-GPU model with separate q/k/v and gate/up linears"
    check_quip_params(quip_params, model.shape)

    def take(key, like):
        t = state_dict[key]
        if tuple(t.shape) != tuple(like.shape):
            raise ValueError(f"{key}: shape {tuple(t.shape)}, expected {tuple(like.shape)}")
        return t

    for i, L in enumerate(model.layers):
        for name, proj in _PROJ.items():
            base, lin = f"{prefix}layers.{i}.{proj}.", L[name]
            if int(state_dict.get(base + "rcp", torch.tensor(0))) != 0:
                raise ValueError(f"{base}rcp != 0: tensor-parallel quantization layout")
            trellis = take(base + "trellis", lin.codes)
            if trellis.dtype != torch.int16:
                raise ValueError(f"{base}trellis: dtype {trellis.dtype}, expected int16")
            lin.codes.copy_(trellis)
            lin.tlut.copy_(take(base + "tlut", lin.tlut).to(torch.float16))
            lin.SU.copy_(take(base + "SU", lin.SU).to(torch.float16))
            lin.SV.copy_(take(base + "SV", lin.SV).float())
            lin.SV32.copy_(lin.SV * 32)
        L["ln1"].copy_(take(f"{prefix}layers.{i}.input_layernorm.weight", L["ln1"]).to(torch.float16))
        L["ln2"].copy_(take(f"{prefix}layers.{i}.post_attention_layernorm.weight", L["ln2"]).to(torch.float16))
        # sign vectors of launches that share one input are kept concatenated
        L["SU_qkv"] = torch.cat([L["q"].SU, L["k"].SU, L["v"].SU]).contiguous()
        L["SU_gu"] = torch.cat([L["gate"].SU, L["up"].SU]).contiguous()
        L["SV_gu"] = torch.cat([L["gate"].SV32, L["up"].SV32]).contiguous()
        L.pop("SV_kv", None)
    model.embed.copy_(take(prefix + "embed_tokens.weight", model.embed).to(torch.float16))
    model.ln_f.copy_(take(prefix + "norm.weight", model.ln_f).to(torch.float16))
    model.lm_head.copy_(take("lm_head.weight", model.lm_head).to(torch.float16))
    model.graph = None        # a captured step holds no copies of the weights, but any cached derived tensors are stale
    return model


def export_state_dict(model, prefix="model."):
    """The inverse of load_state_dict_into: a state dict with upstream's keys, shapes and dtypes (used to build
    synthetic checkpoints for tests; released checkpoints have exactly these entries per layer)."""
    sd = {}
    for i, L in enumerate(model.layers):
        for name, proj in _PROJ.items():
            base, lin = f"{prefix}layers.{i}.{proj}.", L[name]
            sd[base + "trellis"] = lin.codes.clone()
            sd[base + "tlut"] = lin.tlut.clone()
            sd[base + "SU"] = lin.SU.clone()
            sd[base + "SV"] = lin.SV.clone()
            sd[base + "rcp"] = torch.tensor(0)
            sd[base + "tp_rank"] = torch.tensor(8)
        sd[f"{prefix}layers.{i}.input_layernorm.weight"] = L["ln1"].clone()
        sd[f"{prefix}layers.{i}.post_attention_layernorm.weight"] = L["ln2"].clone()
    sd[prefix + "embed_tokens.weight"] = model.embed.clone()
    sd[prefix + "norm.weight"] = model.ln_f.clone()
    sd["lm_head.weight"] = model.lm_head.clone()
    return sd
