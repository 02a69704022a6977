"""The one-pass upload of a checkpoint (weights/upload.py): the tensors a model holds after `Engine.from_folder`
are, bit for bit, those it holds when every checkpoint tensor is read whole and the parts fuse them on the
device; and reading a checkpoint does not keep a second copy of it on the host."""
import json
import os
import subprocess
import sys

import pytest

from helpers import make_folder, tiny

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def held_tensors(model):
    out = {"embedding": model.embedding.table, "head": model.head.weight, "final_norm": model.final_norm.weight}
    for i, block in enumerate(model.blocks):
        out[f"{i}.w_qkv"], out[f"{i}.w_o"] = block.mixer.w_qkv, block.mixer.w_o
        out[f"{i}.q_norm"], out[f"{i}.k_norm"] = block.mixer.q_norm.weight, block.mixer.k_norm.weight
        out[f"{i}.w_gate_up"], out[f"{i}.w_down"] = block.feed_forward.w_gate_up, block.feed_forward.w_down
        out[f"{i}.norm1"], out[f"{i}.norm2"] = block.mixer_norm.weight, block.feed_forward_norm.weight
    return out


@pytest.mark.parametrize("storage", ["bfloat16", "float32"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_uploaded_tensors_equal_the_tensors_fused_on_the_device(tmp_path, name, dtype, storage):
    import qwen3_b200 as q
    cfg = tiny(name)
    folder, _ = make_folder(tmp_path, cfg, seed=5, storage=storage)
    engine = q.Engine.from_folder(folder, dtype=dtype, max_tokens=64)
    compute = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    model = q.build_model(q.load_config(folder).plan())
    model.bind(q.load_weights(folder, model.weight_specs(), model.ignorable_names()), compute, "cuda")
    got, want = held_tensors(engine.model), held_tensors(model)
    assert got.keys() == want.keys()
    arena = engine.weights_arena
    lo, hi = arena.data_ptr(), arena.data_ptr() + arena.numel()
    for key in want:
        assert got[key].dtype == want[key].dtype and got[key].shape == want[key].shape, key
        assert torch.equal(got[key], want[key]), key
        assert lo <= got[key].data_ptr() and got[key].data_ptr() + got[key].numel() * got[key].element_size() <= hi, key
    if cfg["tie_word_embeddings"]:
        assert engine.model.head.weight.data_ptr() == engine.model.embedding.table.data_ptr()


def test_interleaving_and_conversion_by_the_placement_kernel():
    from qwen3_b200.csrc import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    gate = torch.randn(40, 24, generator=g, device="cuda")
    up = torch.randn(40, 24, generator=g, device="cuda")
    want = ops.interleave_gate_up(gate.to(torch.bfloat16), up.to(torch.bfloat16))
    out = torch.zeros(80, 24, dtype=torch.bfloat16, device="cuda")
    ops.place_rows(gate, out, 8, 16, 0)                       # float32 -> bfloat16 on the way
    ops.place_rows(up.to(torch.bfloat16), out, 8, 16, 8)
    assert torch.equal(out, want)
    wide = torch.zeros(90, 24, dtype=torch.float32, device="cuda")
    ops.place_rows(gate.to(torch.bfloat16), wide, 0, 0, 50)   # consecutive rows from row 50, widened exactly
    assert torch.equal(wide[50:], gate.to(torch.bfloat16).float()) and wide[:50].abs().max().item() == 0.0
    with pytest.raises(ops.KernelError):
        ops.place_rows(gate, wide, 0, 0, 60)                  # ten rows too many


LOAD_SCRIPT = r"""
import json, os, resource, sys, time
sys.path.insert(0, sys.argv[1])
import torch
import qwen3_b200 as q
folder, small = sys.argv[2], sys.argv[3]
q.Engine.from_folder(small, dtype="bfloat16", max_tokens=64)      # CUDA context, kernel libraries, pinned-memory pool
torch.cuda.synchronize()
before = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
start = time.time()
engine = q.Engine.from_folder(folder, dtype="bfloat16", max_tokens=64)
torch.cuda.synchronize()
seconds = time.time() - start
after = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
size = os.path.getsize(os.path.join(folder, "model.safetensors"))
print(json.dumps({"grew_bytes": (after - before) * 1024, "file_bytes": size, "seconds": seconds,
                  "device_bytes": engine.weights_arena.numel()}))
"""


def test_loading_holds_no_second_copy_of_the_checkpoint_on_the_host(tmp_path):
    """One layer of the 8B widths with a vocabulary of 20,000 (0.7 GB): the peak resident memory of the process
    grows by a fraction of the file's size (the staging buffers), where a copy of every tensor, or even the
    mapping's own pages left in place, would add all of it."""
    import qwen3_b200 as q
    cfg = dict(tiny("B"), num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=12288, vocab_size=20000, bos_token_id=1, eos_token_id=2)
    folder, _ = make_folder(tmp_path, cfg, seed=1, name="wide")
    small, _ = make_folder(tmp_path, tiny("A"), seed=2, name="small")
    out = subprocess.run([sys.executable, "-c", LOAD_SCRIPT, ROOT, folder, small], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:]
    info = json.loads(out.stdout.strip().splitlines()[-1])
    assert info["file_bytes"] > 600e6
    assert info["grew_bytes"] < 0.4 * info["file_bytes"], info
    assert info["device_bytes"] < 1.01 * info["file_bytes"] + (1 << 20), info      # one arena of the checkpoint's size
