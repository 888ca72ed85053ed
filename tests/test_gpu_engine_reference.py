"""The unmodified reference's Engine (the reference package installed with ``pip install --no-deps --target
baseline/_ref``) driving this package's model, pool and attention backend: a tiny int8 Qwen3 checkpoint written as safetensors + a
Hugging Face config, loaded by the reference's own weight loader (q/k/v and gate/up merged there), one prefill and
four greedy decode steps through ``Engine.forward_batch``; the token ids must be the oracle's.  Skipped where the
reference is not installed."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import attention as oattn
from oracle import fixed_point as ofp
from oracle import linear as olin
from oracle import model as omodel

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
L, HID, HQ, HK, INTER, VOCAB = 2, 256, 4, 2, 512, 1000


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def _write_model(path, rng):
    """Checkpoint under Hugging Face key names (separate q/k/v and gate/up) and the oracle's form of the same weights."""
    from safetensors.torch import save_file
    sd, layers = {}, []

    def lin(key, n, k):
        w = rng.integers(-127, 128, (n, k), dtype=np.int8)
        scale = (rng.uniform(0.25, 0.5, n) * 2.0 ** rng.integers(-3, 0, n)).astype(np.float32)
        sd[key + ".weight"] = torch.from_numpy(w); sd[key + ".weight_scale"] = torch.from_numpy(scale.reshape(n, 1))
        return w, scale

    def merged(parts):
        w = np.concatenate([p[0] for p in parts]); s = np.concatenate([p[1] for p in parts])
        mul, sh = olin.weight_scale_to_mul_shift(s)
        return (w, mul, sh)

    def norm(key, n, lo, hi, fuse=False):
        # the engine casts every non-int8, non-scale tensor to its dtype (bfloat16): draw values that bfloat16 holds
        w = _bf16((rng.integers(128, 256, n) << rng.integers(lo, hi, n)) / 65536.0)
        sd[key + ".weight"] = w.clone()
        if fuse:                                            # q_norm absorbs head_dim ** -0.5, in the weight's dtype
            w = w * (128 ** -0.5)
        return ofp.to_fixed(w.float().numpy())
    for i in range(L):
        p = f"model.layers.{i}."
        q, k, v = lin(p + "self_attn.q_proj", HQ * 128, HID), lin(p + "self_attn.k_proj", HK * 128, HID), lin(p + "self_attn.v_proj", HK * 128, HID)
        o = lin(p + "self_attn.o_proj", HID, HQ * 128)
        g, u, dn = lin(p + "mlp.gate_proj", INTER, HID), lin(p + "mlp.up_proj", INTER, HID), lin(p + "mlp.down_proj", HID, INTER)
        layers.append({"qkv": merged([q, k, v]), "o": merged([o]), "gate_up": merged([g, u]), "down": merged([dn]),
                       "input_norm": norm(p + "input_layernorm", HID, 0, 2), "post_norm": norm(p + "post_attention_layernorm", HID, 0, 2),
                       "q_norm": norm(p + "self_attn.q_norm", 128, 7, 9, fuse=True), "k_norm": norm(p + "self_attn.k_norm", 128, 5, 7)})
    embed = (torch.randn((VOCAB, HID), generator=torch.Generator().manual_seed(3)) * 0.5).to(torch.bfloat16)
    sd["model.embed_tokens.weight"] = embed
    final = norm("model.norm", HID, 0, 2)
    head = merged([lin("lm_head", VOCAB, HID)])
    save_file(sd, os.path.join(path, "model.safetensors"))
    hf = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": HID, "num_attention_heads": HQ,
          "num_key_value_heads": HK, "head_dim": 128, "intermediate_size": INTER, "num_hidden_layers": L, "vocab_size": VOCAB,
          "max_position_embeddings": 128, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "hidden_act": "silu",
          "tie_word_embeddings": False, "torch_dtype": "bfloat16",
          "quantization_config": {"quant_method": "compressed-tensors", "transform_config": {"config_groups": {
              "R4": {"type": "hadamard", "head_dim": 128,
                     "apply": [{"location": "input", "targets": ["re:.*down_proj$"], "inverse": False}]}}}}}
    json.dump(hf, open(os.path.join(path, "config.json"), "w"))
    return {"embed": embed.view(torch.int16).numpy().view(np.uint16), "layers": layers, "final_norm": final, "lm_head": head}


def test_reference_engine_drives_this_package(tmp_path):
    if not os.path.isdir(os.path.join(REF, "minisgl")):
        pytest.skip("the reference is not installed under baseline/_ref")
    rng = np.random.default_rng(17)
    host = _write_model(str(tmp_path), rng)
    steps, P, max_len = 4, 16, 64
    prompt_lens = [5, 17, 32]
    B = len(prompt_lens)
    table = rng.permutation(P)[: B * (max_len // 16)].reshape(B, max_len // 16).astype(np.int32)
    prompts = [rng.integers(0, VOCAB, n).astype(np.int32) for n in prompt_lens]
    json.dump({"prompts": [p.tolist() for p in prompts], "pages": table.tolist(), "num_pages": P, "max_len": max_len},
              open(tmp_path / "case.json", "w"))
    out = tmp_path / "out.npz"
    env = dict(os.environ, MINISGL_INTEGER_MODE="1", PYTHONPATH=ROOT)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_under_reference.py"), REF, str(tmp_path), str(steps), str(out)],
                          env=env, capture_output=True, text=True, timeout=600)
    if proc.returncode != 0 and "ddress already in use" in proc.stderr:
        pytest.skip("the engine's fixed rendezvous port (tcp://127.0.0.1:2333, engine/config.py) is taken on this host")
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    z = np.load(out)
    assert int(z["calls"]) > 0                                       # the sm_100a library did the work
    cache = z["rotary"]

    # ---- oracle: the same prefill and decode steps
    pools = [oattn.PagedKV(P, HK, 128) for _ in range(L)]
    tables = [table[b] for b in range(B)]
    ids = np.concatenate(prompts)
    positions = np.concatenate([np.arange(n) for n in prompt_lens]).astype(np.int32)
    out_loc = np.concatenate([table[b][np.arange(n) // 16] * 16 + np.arange(n) % 16 for b, n in enumerate(prompt_lens)]).astype(np.int32)
    tok, _ = omodel.greedy(ids, host, cache, pools, positions, out_loc, tables, prompt_lens, prompt_lens, HQ, HK, np.cumsum(prompt_lens) - 1)
    want = [tok]
    lens = np.asarray(prompt_lens)
    for _ in range(steps):
        pos = lens.astype(np.int32)
        loc = np.asarray([table[b][pos[b] // 16] * 16 + pos[b] % 16 for b in range(B)], dtype=np.int32)
        lens = lens + 1
        tok, _ = omodel.greedy(tok, host, cache, pools, pos, loc, tables, list(lens), [1] * B, HQ, HK, None)
        want.append(tok)
    np.testing.assert_array_equal(z["tokens"], np.stack(want))
