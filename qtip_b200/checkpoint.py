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
