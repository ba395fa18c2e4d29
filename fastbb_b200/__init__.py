"""fastbb_b200: the ViT block fast path of fastbb, rebuilt for B200 (sm_100a).

    import fastbb_b200 as fastbb
    fastbb.install_vit(model.pretrained, "fh-g0")        # DINOv2-style ViT: get_intermediate_layers -> fast path
    fastbb.install_vit_blocks(timm_vit, "fh-g1")         # any pre-LN ViT block stack: block.forward -> fast path

Spec strings keep the reference's grammar (fastbb/__init__.py:3-18): "<attn>[-g<n>][-graph]" or "off".
  attn  sdpa | ff | fh | hh   accumulate mode of the flash-attention kernel. "sdpa" (the reference's torch-SDPA tier)
                              has no torch path here and runs the fp32-accumulate kernel "ff", which has SDPA-flash
                              precision (fastbb/attention.py:7).
  g0                          fp32 tensor-memory accumulator for every GEMM
  g1                          fp16 accumulator for every GEMM
  g2                          fp16 accumulator except fc2 / w3 (K = 4C), which stays fp32
  g3                          the reference's chunked-fp16 GEMM with fused epilogues; on B200 the fp32 accumulator runs
                              at the fp16 rate, so g3 == g0 here (every mode uses the fused epilogues)
  -graph                      replay the whole stack from one CUDA graph per input shape. The reference only accepts
                              this suffix in models.dinov2.dinov2(); here install_vit() takes it too and
                              install_vit_blocks() ignores it (a single block is too small a unit to graph).
The default spec comes from the FASTBB_VIT environment variable ("fh-g0" if unset), read at import as in the reference.
"""
import os

DEFAULT_VIT = os.environ.get("FASTBB_VIT", "fh-g0")

_ATTN = ("sdpa", "ff", "fh", "hh")
_GACC = {"g0": False, "g1": True, "g2": "nofc2", "g3": "chunk", "": False}


def split_graph_suffix(spec):
    """'hh-g1-graph' -> ('hh-g1', True); 'hh-g1' -> ('hh-g1', False)."""
    if spec.endswith("-graph"):
        return spec[: -len("-graph")], True
    return spec, False


def parse_vit_spec(spec):
    """'<attn>-g<n>' -> (attn, gacc) with gacc False (g0) | True (g1) | 'nofc2' (g2) | 'chunk' (g3), exactly the pair the
    reference's parser returns (fastbb/__init__.py:15-18). A trailing '-graph' is accepted and dropped; unknown names
    raise KeyError like the reference's dict lookup, unknown attention names raise ValueError."""
    spec, _ = split_graph_suffix(spec)
    attn, _, g = spec.partition("-")
    gacc = _GACC[g]
    if attn not in _ATTN:
        raise ValueError(f"unknown attention variant {attn!r} in spec {spec!r}: expected one of {_ATTN}")
    return attn, gacc


def install_vit(vit, spec=None, out_dtype=None):
    """Route `vit.get_intermediate_layers` through the B200 kernels (weights become fp16 in place).
    Returns the FastViT, or None for spec "off" (the module is left untouched). Mirrors fastbb/__init__.py:21-28."""
    spec = spec or DEFAULT_VIT
    if spec == "off":
        return None
    from .vit import FastViT
    spec, graphs = split_graph_suffix(spec)
    attn, gacc = parse_vit_spec(spec)
    return FastViT(vit, attn=attn, gacc=gacc, out_dtype=out_dtype, graphs=graphs).install()


def install_vit_blocks(model, spec=None, convert=True):
    """Patch the forward of every supported pre-LN transformer block inside `model`; returns how many were patched.
    Mirrors fastbb/__init__.py:31-34 / fastbb/vit.py:311-328."""
    from .vit import install_vit_blocks as _install
    return _install(model, spec or DEFAULT_VIT, convert)
