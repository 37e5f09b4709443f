"""Model presets shared by the four schedule families.

The reference keeps one `transformer_configs` dict per family file
(gpt_fast/gpt_ladder_TP.py:65-207, gpt_dense_TP.py:63-182, gpt_parallel_TP.py:63-133,
gpt_desync_TP.py:68-249) with mostly equal entries.  Here every architecture is written once
and each family lists which names it offers and which schedule flags it attaches, so that
`family:preset` strings accepted by the reference's benchmark driver resolve to the same shapes.
Two presets are added for shapes the reference does not have (8 KV heads for the 1B and 405B
Ladder-Llama shapes).
"""
from copy import deepcopy

_LLAMA31_SCALING = dict(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)


def _arch(n_layer, n_head, dim, **kw):
    return dict(n_layer=n_layer, n_head=n_head, dim=dim, **kw)


def _star(n_layer, n_head, dim, inter):
    # StarCoder-style research shapes: MHA, vocab 49152, 2k context
    return _arch(n_layer, n_head, dim, block_size=2048, n_local_heads=n_head, intermediate_size=inter,
                 vocab_size=49152, rope_base=10000)


def _llama3(n_layer, n_head, dim, inter, **kw):
    return _arch(n_layer, n_head, dim, block_size=8192, n_local_heads=8, intermediate_size=inter,
                 vocab_size=128256, rope_base=500000, **kw)


ARCH = {
    "CodeLlama-7b-Python-hf": _arch(32, 32, 4096, block_size=16384, vocab_size=32000, rope_base=1000000),
    "1b": _star(40, 24, 1536, 4096),
    "1.55b": _star(52, 24, 1536, 4096),
    "3b": _star(40, 32, 2304, 9216),
    "3b-36h": _star(40, 36, 2304, 9216),
    "3.9bh": _star(52, 32, 2304, 9216),
    "3.9bw1": _star(40, 32, 3200, 9216),
    "3.9bw2": _star(40, 32, 2560, 11000),
    "7B": _arch(32, 32, 4096),
    "13B": _arch(40, 40, 5120),
    "30B": _arch(60, 52, 6656),
    "34B": _arch(48, 64, 8192, vocab_size=32000, n_local_heads=8, intermediate_size=22016, rope_base=1000000),
    "70B": _arch(80, 64, 8192, n_local_heads=8, intermediate_size=28672),
    "Mistral-7B": _arch(32, 32, 4096, n_local_heads=8, intermediate_size=14336, vocab_size=32000),
    "stories15M": _arch(6, 6, 288),
    "stories110M": _arch(12, 12, 768),
    "llama-3.2-1b": _arch(16, 32, 2048, intermediate_size=8192, vocab_size=128256),
    "llama-3.2-3b": _arch(28, 24, 3072, intermediate_size=8192, vocab_size=128256),
    "llama-3-8b": _llama3(32, 32, 4096, 14336),
    "llama-3-8b-4layers": _llama3(4, 32, 4096, 14336),
    "llama-3-70b": _llama3(80, 64, 8192, 28672),
    "llama-3.1-405b": _arch(126, 128, 16384, block_size=131072, n_local_heads=16, intermediate_size=53248,
                            vocab_size=128256, rope_base=500000, rope_scaling=_LLAMA31_SCALING),
    "bloom-176b": _arch(70, 112, 14336, block_size=8192, n_local_heads=112, intermediate_size=50176,
                        vocab_size=250880, rope_base=500000),
    # shapes of the headline benchmark that the reference's presets do not cover
    "ladder-llama-1b": _arch(16, 32, 2048, block_size=2048, n_local_heads=8, intermediate_size=8192,
                             vocab_size=128256, rope_base=500000),
    "ladder-llama-405b-kv8": _arch(126, 128, 16384, block_size=131072, n_local_heads=8, intermediate_size=53248,
                                   vocab_size=128256, rope_base=500000, rope_scaling=_LLAMA31_SCALING),
}

_COMMON = ["CodeLlama-7b-Python-hf", "1b", "3b", "7B", "13B", "30B", "34B", "70B", "Mistral-7B", "stories15M",
           "stories110M", "llama-3.2-1b", "llama-3.2-3b", "llama-3-8b", "llama-3-70b", "llama-3.1-405b",
           "ladder-llama-1b", "ladder-llama-405b-kv8"]
_WIDE = ["3.9bh", "3.9bw1", "3.9bw2"]


def _no_reduce(n_layer):
    return [{"attention": False, "mlp": False} for _ in range(n_layer)]


def _every_other_mlp(n_layer):
    return [{"attention": False, "mlp": False}, {"attention": False, "mlp": True}] * (n_layer // 2)


def family_presets(family):
    """Returns {preset name: ModelArgs kwargs} for 'ladder', 'dense', 'parallel' or 'desync'."""
    out = {}

    def add(name, arch=None, **extra):
        cfg = deepcopy(ARCH[arch or name])
        cfg.update(extra)
        out[name] = cfg

    names = list(_COMMON)
    if family in ("ladder", "dense"):
        names += _WIDE
    if family == "ladder":
        names += ["1.55b", "bloom-176b"]
    if family == "dense":
        names += ["llama-3-8b-4layers"]
    for n in names:
        add(n)
    add("70B-semi-compiled", "70B", semi_compiled_model=True)
    if family == "ladder":
        add("llama-3-8b-semi-compiled", "llama-3-8b", semi_compiled_model=True)
        add("llama-3-70b-semi-compiled", "llama-3-70b", semi_compiled_model=True)
    if family == "desync":
        # In the reference's desync table the plain "1b" entry carries the no-reduce pattern and
        # "1b-upper-bound" the default one; "3b" uses 36 heads.  Kept as they are.
        add("1b", "1b", reduce_pattern=_no_reduce(40), force_disable_last_all_reduce=True)
        add("1b-upper-bound", "1b")
        add("3b", "3b-36h")
        add("3b-upper-bound", "3b-36h", reduce_pattern=_no_reduce(40), force_disable_last_all_reduce=True)
        add("70B-infinite", "70B", reduce_pattern=_no_reduce(80))
        add("70B-infinite-semi-compiled", "70B", semi_compiled_model=True, reduce_pattern=_no_reduce(80))
        for base, layers in (("llama-3-8b", 32), ("llama-3-70b", 80)):
            add(base + "-4x", base, reduce_pattern=_every_other_mlp(layers))
            add(base + "-upper-bound", base, reduce_pattern=_no_reduce(layers), force_disable_last_all_reduce=True)
        add("llama-3-8b-infinite", "llama-3-8b", reduce_pattern=_no_reduce(32))
        add("llama-3.1-405b-upper-bound", "llama-3.1-405b", reduce_pattern=_no_reduce(126),
            force_disable_last_all_reduce=True)
        add("ladder-llama-405b-kv8-upper-bound", "ladder-llama-405b-kv8", reduce_pattern=_no_reduce(126),
            force_disable_last_all_reduce=True)
    return out
