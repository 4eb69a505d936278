"""Makes the golden logits of tests/golden/*.npz by running the reference's own model
code (axonn-ai/yalis, yalis/external/model.py ``GPT``) on the CPU in float32.

Run once, where the reference is mounted:

    python tests/golden/make_golden.py /path/to/axonn-ai-yalis

The reference cannot be imported as shipped here (axonn, litgpt and lightning are not
installed), so this script imports ``yalis`` as a namespace package (skipping its
``__init__``, which pulls in the engine) and provides three stand-ins for modules the
model file imports but the single-GPU dense path never calls: ``axonn`` (group sizes of 1,
identity Drop/Gather), ``yalis.tensor_parallel`` (placeholders) and ``litgpt.model``
(aliased to the reference's own model file, which is where its RMSNorm lives).

For each tiny configuration it writes the same seeded random weights the tests use,
re-lays them out the way the reference stores them (QKV grouped per KV group,
gate/up rows interleaved: yalis/external/convert_hf_checkpoint.py:791-796, 833-835),
runs (1) one whole prompt as PREFILL and (2) a prefix as PREFILL followed by
DECODE_SINGLE tokens, and stores the logits together with the weights themselves
(under ``w/<tensor name>``, as the 16 bits of their bfloat16 values, which is what the
model file holds), so that the comparison never depends on how a torch build draws
random numbers.  tests/test_plain.py compares the plain implementation with these files.
"""

import hashlib
import os
import sys
import tempfile
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def install_stand_ins(reference_root: str) -> None:
    pkg = types.ModuleType("yalis")
    pkg.__path__ = [os.path.join(reference_root, "yalis")]
    sys.modules["yalis"] = pkg

    class _Identity:
        @staticmethod
        def apply(x, *a, **k):
            return x

    ax_pkg = types.ModuleType("axonn")
    ax_pkg.__path__ = []
    ax = types.ModuleType("axonn.axonn")
    ax.config = types.SimpleNamespace(G_intra_r=1, G_intra_c=1, G_intra_d=1)
    ax.comm_handle = types.SimpleNamespace(inner_intra_layer_parallel_group=None)
    ax_pkg.axonn = ax
    intra = types.ModuleType("axonn.intra_layer")
    intra.__path__ = []
    comm = types.ModuleType("axonn.intra_layer.communication")
    comm.Drop, comm.Gather = _Identity, _Identity
    intra.communication = comm
    sys.modules.update({"axonn": ax_pkg, "axonn.axonn": ax, "axonn.intra_layer": intra,
                        "axonn.intra_layer.communication": comm})
    tp = types.ModuleType("yalis.tensor_parallel")
    tp.TPLinear = tp.TPMoE = tp.TPRMSNorm = type("Unused", (), {})
    sys.modules["yalis.tensor_parallel"] = tp
    import yalis.external.model as ref_model
    lit = types.ModuleType("litgpt")
    lit.__path__ = []
    lit.model = ref_model
    sys.modules.update({"litgpt": lit, "litgpt.model": ref_model})


def reference_state_dict(weights, cfg):
    """HF-named tensors -> the reference's parameter names and layouts."""
    nh, g, hs = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per = nh // g
    sd = {"transformer.wte.weight": weights["model.embed_tokens.weight"],
          "transformer.ln_f.weight": weights["model.norm.weight"]}
    head = "model.embed_tokens.weight" if cfg["tie_word_embeddings"] else "lm_head.weight"
    sd["lm_head.weight"] = weights[head]
    for l in range(cfg["num_hidden_layers"]):
        p, o = f"model.layers.{l}.", f"transformer.h.{l}."
        q = weights[p + "self_attn.q_proj.weight"].view(g, per * hs, -1)
        k = weights[p + "self_attn.k_proj.weight"].view(g, hs, -1)
        v = weights[p + "self_attn.v_proj.weight"].view(g, hs, -1)
        sd[o + "attn.attn.weight"] = torch.cat([q, k, v], dim=1).reshape((nh + 2 * g) * hs, -1)
        sd[o + "attn.proj.weight"] = weights[p + "self_attn.o_proj.weight"]
        gate, up = weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"]
        sd[o + "mlp.gate_up_proj.weight"] = torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], -1)
        sd[o + "mlp.proj.weight"] = weights[p + "mlp.down_proj.weight"]
        sd[o + "norm_1.weight"] = weights[p + "input_layernorm.weight"]
        sd[o + "norm_2.weight"] = weights[p + "post_attention_layernorm.weight"]
    return sd


def weights_checksum(weights) -> str:
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].contiguous().numpy().tobytes())
    return h.hexdigest()


def run(which: str, n_tokens: int, prefix: int, std: float):
    import plain_llama as plain
    from tiny import TINY
    from yalis.attention.backends import AttentionBackend
    from yalis.constants import EnginePhase
    from yalis.external.config import Config
    from yalis.external.model import GPT
    from yalis_b200.config.presets import preset
    from yalis_b200.weights.loader import write_random_model

    name, seed, _ = TINY[which]
    with tempfile.TemporaryDirectory() as d:
        write_random_model(preset(name), d, seed=seed, std=std)
        cfg, weights = plain.read_config(d), plain.read_weights(d)
    scaling = cfg["rope_scaling"]
    config = Config(
        name="golden", block_size=cfg["max_position_embeddings"], n_layer=cfg["num_hidden_layers"],
        n_embd=cfg["hidden_size"], vocab_size=cfg["vocab_size"], padded_vocab_size=cfg["vocab_size"],
        n_head=cfg["num_attention_heads"], n_query_groups=cfg["num_key_value_heads"], head_size=cfg["head_dim"],
        rotary_percentage=1.0, parallel_residual=False, bias=False, norm_class_name="RMSNorm",
        norm_eps=cfg["rms_norm_eps"], mlp_class_name="LLaMAMLP", intermediate_size=cfg["intermediate_size"],
        rope_base=int(cfg["rope_theta"]),
        rope_adjustments=None if scaling is None else dict(
            factor=scaling["factor"], low_freq_factor=scaling["low_freq_factor"],
            high_freq_factor=scaling["high_freq_factor"],
            original_max_seq_len=scaling["original_max_position_embeddings"]))
    config.tensor_parallel = False
    config.use_intra_head_parallelism = False
    config.attention_backend = AttentionBackend.SDPA
    config.use_paged_kv_caching = False
    config.prestore_kv_cache = True
    config.init_device = "cpu"
    config.dtype = torch.float32
    model = GPT(config).to(torch.float32).eval()
    model.load_state_dict(reference_state_dict(weights, cfg), strict=True)
    gen = torch.Generator().manual_seed(100 + seed)
    tokens = torch.randint(0, cfg["vocab_size"], (n_tokens,), generator=gen)
    with torch.no_grad():
        model.set_kv_cache(1, device="cpu", dtype=torch.float32)
        counter = torch.zeros(1, dtype=torch.int32)
        whole = model(tokens[None], EnginePhase.PREFILL, torch.tensor([n_tokens]), None, counter)["logits"][0]
        model.set_kv_cache(1, device="cpu", dtype=torch.float32)
        counter = torch.zeros(1, dtype=torch.int32)
        model(tokens[None, :prefix], EnginePhase.PREFILL, torch.tensor([prefix]), None, counter)
        steps = []
        for t in range(prefix, n_tokens):
            counter = torch.tensor([t], dtype=torch.int32)
            out = model(tokens[None, t:t + 1], EnginePhase.DECODE_SINGLE, None, None, counter)["logits"][0, 0]
            steps.append(out)
        decoded = torch.stack(steps)
    out = os.path.join(HERE, f"tiny_{which}.npz")
    stored = {}
    for wname, t in weights.items():
        as_bf16 = t.to(torch.bfloat16)
        assert torch.equal(as_bf16.float(), t.float()), f"{wname} is not representable in bfloat16"
        stored["w/" + wname] = as_bf16.view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(out, tokens=tokens.numpy(), whole=whole.numpy().astype(np.float32),
                        decoded=decoded.numpy().astype(np.float32), prefix=np.int64(prefix), std=np.float64(std),
                        weights_sha256=np.array(weights_checksum(weights)), **stored)
    print(f"{out}: whole {tuple(whole.shape)}, decoded {tuple(decoded.shape)}, "
          f"whole-vs-decoded max abs {float((whole[prefix:] - decoded).abs().max()):.3e}")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <checkout of the reference>")
    install_stand_ins(sys.argv[1])
    run("A", n_tokens=24, prefix=17, std=0.1)
    run("B", n_tokens=40, prefix=33, std=0.1)
