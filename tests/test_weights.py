"""Weight files: strict loading errors and the random-weights mode (no GPU)."""
import json
import struct

import numpy as np
import pytest
import torch

import burn_transformers_b200 as bt
from burn_transformers_b200.config import architecture_for, config_from_folder
from burn_transformers_b200.errors import CheckpointError
from burn_transformers_b200.weights import check, discover, load_weights
from burn_transformers_b200.weights import safetensors_io as st
from tiny_configs import TINY_A, TINY_B, make_folder


def plan_of(folder):
    arch, config = config_from_folder(folder)
    return arch.build(config).weights


def rewrite(folder, edit):
    path = folder / "model.safetensors"
    tensors = {n: st.read_tensor(e) for n, e in st.read_header(path).items()}
    edit(tensors)
    st.write_file(path, tensors)


def test_random_folder_loads_and_is_deterministic(tmp_path):
    a = make_folder(tmp_path / "a", TINY_A, seed=7, storage="bfloat16", loud=False)
    b = make_folder(tmp_path / "b", TINY_A, seed=7, storage="bfloat16", loud=False)
    c = make_folder(tmp_path / "c", TINY_A, seed=8, storage="bfloat16", loud=False)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    tensors, report = load_weights(a, plan_of(a), "bfloat16", "cpu")
    assert tensors["wte.weight"].dtype == torch.bfloat16          # matrices in the compute dtype
    assert tensors["ln_f.weight"].dtype == torch.float32          # a tensor stored in 32-bit stays so
    assert tensors["h.0.attn.c_attn.bias"].dtype == torch.float32
    assert {r["name"] for r in report} == set(plan_of(a).tensors)
    t32, _ = load_weights(a, plan_of(a), "float32", "cpu")
    assert all(t.dtype == torch.float32 for t in t32.values())
    # the reference's distributions: std 0.02, residual writers 0.02/sqrt(2L), zero biases, unit gains
    assert abs(float(t32["wte.weight"].std()) - 0.02) < 2e-3
    assert abs(float(t32["h.0.mlp.c_proj.weight"].std()) - 0.02 / 2.0) < 2e-3
    assert float(t32["h.1.attn.c_attn.bias"].abs().max()) == 0.0
    assert float((t32["h.1.ln_1.weight"] - 1).abs().max()) == 0.0


def test_missing_unexpected_and_wrong_shape_in_one_error(tmp_path):
    folder = make_folder(tmp_path, TINY_A)

    def edit(t):
        del t["h.1.ln_2.bias"]
        del t["wpe.weight"]
        t["h.0.extra.weight"] = torch.zeros(3)
        t["h.0.mlp.c_fc.weight"] = torch.zeros(64, 255)
        t["ln_f.bias"] = torch.zeros(64, dtype=torch.int32)
    rewrite(folder, edit)
    with pytest.raises(CheckpointError) as info:
        check(plan_of(folder), discover(folder))
    e = info.value
    assert e.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert e.unexpected == ["h.0.extra.weight"]
    assert len(e.mismatched) == 2 and "h.0.mlp.c_fc.weight" in e.mismatched[0] and "[64, 255]" in e.mismatched[0]
    assert "ln_f.bias" in e.mismatched[1] and "I32" in e.mismatched[1]
    for text in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape or dtype (2)"):
        assert text in str(e)


def test_namespaces_legacy_buffers_and_tied_head(tmp_path):
    folder = make_folder(tmp_path, TINY_B)

    def edit(t):
        for name in list(t):
            t["transformer." + name] = t.pop(name)
        t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)
        t["transformer.h.2.attn.masked_bias"] = torch.tensor(-1e4)
        t["lm_head.weight"] = t["transformer.wte.weight"].clone()
    rewrite(folder, edit)
    prefix, entries = check(plan_of(folder), discover(folder))
    assert prefix == "transformer." and "wte.weight" in entries
    rewrite(folder, lambda t: t["lm_head.weight"].add_(1.0))
    with pytest.raises(CheckpointError, match="tied tensor"):
        check(plan_of(folder), discover(folder))

    def both(t):
        del t["lm_head.weight"]
        t["wte.weight"] = t["transformer.wte.weight"].clone()
    rewrite(folder, both)
    with pytest.raises(CheckpointError, match="namespace"):
        check(plan_of(folder), discover(folder))


def test_broken_files(tmp_path):
    folder = make_folder(tmp_path, TINY_A)
    path = folder / "model.safetensors"
    blob = path.read_bytes()
    with pytest.raises(CheckpointError, match="no model.safetensors"):
        discover(tmp_path / "nowhere")
    path.write_bytes(blob[:-100])
    with pytest.raises(CheckpointError, match="truncated"):
        discover(folder)
    path.write_bytes(blob[:4])
    with pytest.raises(CheckpointError, match="truncated"):
        discover(folder)
    path.write_bytes(struct.pack("<Q", 10 ** 12) + blob[8:])
    with pytest.raises(CheckpointError, match="invalid header length"):
        discover(folder)
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + n])
    header["wte.weight"]["data_offsets"][1] += 4
    raw = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + blob[8 + n:])
    with pytest.raises(CheckpointError, match="invalid data offsets"):
        discover(folder)


def test_sharded_index(tmp_path):
    folder = make_folder(tmp_path, TINY_A)
    path = folder / "model.safetensors"
    tensors = {n: st.read_tensor(e) for n, e in st.read_header(path).items()}
    names = sorted(tensors)
    half = len(names) // 2
    st.write_file(folder / "model-00001-of-00002.safetensors", {n: tensors[n] for n in names[:half]})
    st.write_file(folder / "model-00002-of-00002.safetensors", {n: tensors[n] for n in names[half:]})
    path.unlink()
    weight_map = {n: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
                  for i, n in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    loaded, _ = load_weights(folder, plan_of(folder), "float32", "cpu")
    assert torch.equal(loaded["wte.weight"], tensors["wte.weight"])


def test_loud_weights_move_every_tensor(tmp_path):
    folder = make_folder(tmp_path, TINY_A, loud=True)
    t, _ = load_weights(folder, plan_of(folder), "float32", "cpu")
    assert float(t["h.0.attn.c_attn.bias"].abs().max()) > 0
    assert float((t["ln_f.weight"] - 1).abs().max()) > 0
    assert float(t["h.0.attn.c_attn.weight"].std()) > 0.1


# ---- tensors that are made from stored tensors: Stored(transposed), Split, Concat ---------------------------------

def split_qkv_plan(folder):
    """GPT-2's plan for a checkpoint that stores queries, keys and values separately and every projection [out, in]
    (the layout most other decoders' checkpoints have): only the sources differ, the parts are the same."""
    from burn_transformers_b200.weights.spec import Concat, Stored
    arch, config = config_from_folder(folder)
    model = arch.build(config)
    for i in range(config.n_layer):
        p = f"h.{i}."
        model.sources[p + "attn.c_attn.weight"] = Concat(tuple(Stored(p + f"attn.{x}.weight", transposed=True) for x in "qkv"), axis=1)
        model.sources[p + "attn.c_attn.bias"] = Concat(tuple(Stored(p + f"attn.{x}.bias") for x in "qkv"), axis=0)
        model.sources[p + "attn.c_proj.weight"] = Stored(p + "attn.o.weight", transposed=True)
        model.sources[p + "mlp.c_fc.weight"] = Stored(p + "mlp.up.weight", transposed=True)
    return model


def store_split(folder):
    """Rewrites a GPT-2 folder's file in the layout of `split_qkv_plan`."""
    def edit(t):
        for name in [n for n in t if n.endswith("attn.c_attn.weight")]:
            p = name[:-len("attn.c_attn.weight")]
            w, b = t.pop(name), t.pop(p + "attn.c_attn.bias")
            d = w.shape[0]
            for j, x in enumerate("qkv"):
                t[p + f"attn.{x}.weight"] = w[:, j * d:(j + 1) * d].t().contiguous()
                t[p + f"attn.{x}.bias"] = b[j * d:(j + 1) * d].contiguous()
            t[p + "attn.o.weight"] = t.pop(p + "attn.c_proj.weight").t().contiguous()
            t[p + "mlp.up.weight"] = t.pop(p + "mlp.c_fc.weight").t().contiguous()
    rewrite(folder, edit)


def test_separate_transposed_projections_load_into_the_same_parts(tmp_path):
    fused = make_folder(tmp_path / "fused", TINY_B, seed=5, storage="float32", loud=True)
    split = make_folder(tmp_path / "split", TINY_B, seed=5, storage="float32", loud=True)
    store_split(split)
    want, _ = load_weights(fused, plan_of(fused), "float32", "cpu")
    plan = split_qkv_plan(split).weights
    got, report = load_weights(split, plan, "float32", "cpu")
    assert set(got) == set(want) and all(torch.equal(got[n], want[n]) for n in want)
    assert all(t.is_contiguous() for t in got.values())
    actions = {r["name"]: r["action"] for r in report}
    assert actions["h.0.attn.c_attn.weight"] == "concat" and actions["h.0.attn.c_proj.weight"] == "transpose"
    assert actions["wte.weight"] == "map"
    # the strict accounting is kept, in the checkpoint's own names
    with pytest.raises(CheckpointError) as info:
        check(plan_of(fused), discover(split))
    assert "h.0.attn.q.weight" in info.value.unexpected and "h.0.attn.c_attn.weight" in info.value.missing
    rewrite(split, lambda t: (t.pop("h.1.attn.k.bias"), t.__setitem__("h.2.attn.v.weight", torch.zeros(96, 95))))
    with pytest.raises(CheckpointError) as info:
        check(plan, discover(split))
    assert info.value.missing == ["h.1.attn.k.bias"]
    assert any(m.startswith("h.2.attn.v.weight: expected shape [96, 96]") for m in info.value.mismatched)


def test_split_reads_pieces_of_one_stored_tensor():
    from burn_transformers_b200.weights.spec import MATRIX, Concat, Split, Stored, TensorSpec, WeightPlan, resolve
    plan = WeightPlan({"q": TensorSpec((4, 6)), "k": TensorSpec((4, 2)), "v": TensorSpec((4, 2))},
                      sources={"q": Split("qkv", 1, (6, 2, 2), 0), "k": Split("qkv", 1, (6, 2, 2), 1),
                               "v": Split("qkv", 1, (6, 2, 2), 2)})
    assert {n: s.shape for n, s in plan.stored().items()} == {"qkv": (4, 10)}
    stored = {"qkv": torch.arange(40.0).reshape(4, 10)}
    assert torch.equal(resolve(plan.source_of("k"), stored), stored["qkv"][:, 6:8])
    # stored the other way round: [10, 4]
    flipped = WeightPlan({"k": TensorSpec((4, 2))}, sources={"k": Split("qkv_t", 1, (6, 2, 2), 1, transposed=True)})
    assert flipped.stored()["qkv_t"].shape == (10, 4)
    assert torch.equal(resolve(flipped.source_of("k"), {"qkv_t": stored["qkv"].t().contiguous()}), stored["qkv"][:, 6:8])
    # two readers that disagree about a stored tensor's shape are a fault of the plan
    bad = WeightPlan({"a": TensorSpec((4, 6)), "b": TensorSpec((4, 3))},
                     sources={"a": Split("x", 1, (6, 2), 0), "b": Split("x", 1, (3, 3), 0)})
    with pytest.raises(ValueError, match="is asked for as"):
        bad.stored()
    with pytest.raises(ValueError, match="cannot make"):
        WeightPlan({"a": TensorSpec((4, 7))}, sources={"a": Concat((Stored("p"), Stored("q")), 1)}).stored()


def test_the_random_model_program_writes_the_folder_the_library_writes(tmp_path):
    """bin/random_model: the same configuration and seed give the file `write_random_model` gives; a configuration
    that cannot be built ends with one line on standard error and a non-zero exit, not a traceback."""
    import subprocess
    import sys
    from pathlib import Path
    program = Path(__file__).resolve().parent.parent / "bin" / "random_model"
    config = dict(TINY_A)
    (tmp_path / "c.json").write_text(json.dumps(config))
    done = subprocess.run([sys.executable, str(program), str(tmp_path / "c.json"), str(tmp_path / "a"), "--seed", "5", "--loud"],
                          capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stderr
    assert done.stdout.strip() == str(tmp_path / "a")
    bt.write_random_model(tmp_path / "b", config, 5, loud=True)
    assert (tmp_path / "a" / "model.safetensors").read_bytes() == (tmp_path / "b" / "model.safetensors").read_bytes()
    assert json.loads((tmp_path / "a" / "config.json").read_text()) == json.loads((tmp_path / "b" / "config.json").read_text())
    bad = subprocess.run([sys.executable, str(program), json.dumps(dict(config, n_head=5)), str(tmp_path / "c")],
                         capture_output=True, text=True, timeout=300)
    assert bad.returncode == 1 and bad.stderr.startswith("random_model: gpt2.n_head") and "Traceback" not in bad.stderr
