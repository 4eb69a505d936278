"""The plain implementation against the reference's own model code (golden files made
by tests/golden/make_golden.py from yalis/external/model.py on the CPU), and against
itself under a few identities."""

import hashlib
import os
import tempfile

import numpy as np
import pytest
import torch

import plain_llama as plain
from tiny import TINY
from yalis_b200.config.presets import preset
from yalis_b200.weights.loader import write_random_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _checksum(weights):
    h = hashlib.sha256()
    for name in sorted(weights):
        h.update(name.encode())
        h.update(weights[name].contiguous().numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("which", ["A", "B"])
def test_plain_matches_reference_model(which):
    """The golden file holds the weights the reference's model ran with, so nothing here depends on how this
    torch build draws random numbers."""
    g = np.load(os.path.join(GOLDEN, f"tiny_{which}.npz"))
    name, seed, _ = TINY[which]
    cfg = plain.normalise_config(preset(name))
    weights = {k[2:]: torch.from_numpy(g[k].view(np.int16).copy()).view(torch.bfloat16).float()
               for k in g.files if k.startswith("w/")}
    assert weights and _checksum(weights) == str(g["weights_sha256"])
    with tempfile.TemporaryDirectory() as d:             # and the loader's view of the same model folder agrees
        write_random_model(preset(name), d, seed=seed, std=float(g["std"]))
        fresh = plain.read_weights(d)
    assert set(fresh) == set(weights) and all(fresh[k].shape == weights[k].shape for k in weights)
    tokens = g["tokens"].tolist()
    ours = plain.forward_logits(tokens, weights, cfg).numpy()
    scale = np.abs(g["whole"]).max()
    assert np.abs(ours - g["whole"]).max() <= 2e-5 * scale
    # the reference's own token-by-token decoding lands on the same logits
    prefix = int(g["prefix"])
    assert np.abs(ours[prefix:] - g["decoded"]).max() <= 2e-5 * scale


def test_rope_frequencies_three_regimes():
    cfg = plain.normalise_config(preset("tiny-B"))
    plain_inv = plain.rope_inverse_frequencies(cfg["head_dim"], cfg["rope_theta"], None)
    scaled = plain.rope_inverse_frequencies(cfg["head_dim"], cfg["rope_theta"], cfg["rope_scaling"])
    ratio = (scaled / plain_inv).numpy()
    factor = cfg["rope_scaling"]["factor"]
    assert np.isclose(ratio[0], 1.0)                       # high frequencies untouched
    assert np.isclose(ratio[-1], 1.0 / factor)             # low frequencies divided by the factor
    assert ((ratio > 1.0 / factor + 1e-6) & (ratio < 1.0 - 1e-6)).any()   # and a smoothed band between


def test_attention_prefix_invariance():
    """Causal attention: the output at position t does not depend on later tokens."""
    torch.manual_seed(0)
    q, k, v = torch.randn(9, 4, 16), torch.randn(9, 2, 16), torch.randn(9, 2, 16)
    pos = torch.arange(9)
    full = plain.causal_attention(q, k, v, pos, pos)
    part = plain.causal_attention(q[:5], k[:5], v[:5], pos[:5], pos[:5])
    assert torch.allclose(full[:5], part, atol=1e-6)
    win = plain.causal_attention(q, k, v, pos, pos, window=3)
    last = plain.causal_attention(q[8:], k[6:], v[6:], pos[8:], pos[6:])
    assert torch.allclose(win[8:], last, atol=1e-6)


def test_sampling_distribution_rules():
    logits = torch.tensor([2.0, 1.0, 0.5, -1.0, 0.0])
    p = plain.sampling_distribution(logits, 1.0, None, 1.0)
    assert torch.allclose(p, torch.softmax(logits, 0))
    p = plain.sampling_distribution(logits, 1.0, 2, 1.0)
    assert (p > 0).sum() == 2 and p[0] > p[1] > 0
    p = plain.sampling_distribution(logits, 0.5, None, 0.6)     # the first alone passes 0.6 at T=0.5
    assert (p > 0).sum() == 1 and p[0] == 1.0
    p = plain.sampling_distribution(logits, 1.0, None, 0.0)     # top_p 0 keeps the first only
    assert (p > 0).sum() == 1


def test_greedy_generate_is_argmax_chain():
    with tempfile.TemporaryDirectory() as d:
        write_random_model(preset("tiny-A"), d, seed=0, std=0.3)
        cfg, w = plain.read_config(d), plain.read_weights(d)
    out = plain.greedy_generate([3, 1, 4, 1, 5], 3, w, cfg)
    seq = [3, 1, 4, 1, 5]
    for t in out:
        assert t == int(plain.forward_logits(seq, w, cfg)[-1].argmax())
        seq.append(t)
