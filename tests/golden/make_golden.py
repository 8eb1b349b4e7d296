"""Writes tests/golden/reference_vectors.json from the reference's own test
fixtures, so that the suite can run where the reference tree is not mounted.

Sources (paths within presk-lang/presk, read as text):
  tests/run/layernorm_apply.snap, rmsnorm_apply.snap   seed-0 outputs of the exact interpreter, 12 digits
  tests/run/mlp_mse.snap, mlp_mse_grad.snap             seed-0 loss and gradient of examples/spec/mlp/mlp.psk at D = 4, B = 2
  tests/run/rope_attention2.snap, rope_attention3.snap   seed-0 outputs of examples/spec/rope/rope.psk `attention2`, `attention3` at B = 2, T = 8
  tests/run/stack_grad.snap                             seed-0 gradient of examples/tests/data/stack_grad.psk `loss_grad` at B = 2
  tests/run/concat_loss.snap, concat_loss_grad.snap     seed-0 loss and gradient of examples/spec/concat/concat.psk at B = 2, T = 8
  crates/presk-interp/src/key.rs:86-93                  the first four normal draws of the key seed 0 names
  crates/presk-kernel/tests/snapshots/conformance__linear_kernels.snap
                                                        the kernel text of a row-wise `dot` and an `add` (what an executor is handed)
  tests/run/minigpt_forward.snap, minigpt_loss.snap      seed-0 logits (all zero: the head is initialised to zeros) and loss of MiniGPT
  examples/tests/data/windows.psk.d, examples/tests/train/reg.psk.d, examples/tutorial/data/pairs.psk.d,
  examples/spec/minigpt/data/tokens.psk.d                the reference's own small data files (version 1), whole, with
                                                        their sample types and leaves (written to data_files.json)
Run:  python tests/golden/make_golden.py <path of the reference's tree>
"""
import json
import os
import re
import sys

if len(sys.argv) < 2:
    sys.exit(__doc__)
ref = sys.argv[1]
out = {}
for name in ("layernorm_apply", "rmsnorm_apply"):
    text = open(os.path.join(ref, "tests", "run", name + ".snap")).read()
    body = text.split("---")[-1]
    m = re.search(r"\[batch: (\d+), model: (\d+)\] (\[\[.*\]\])", body)
    out[name] = {"shape": [int(m.group(1)), int(m.group(2))], "values": json.loads(m.group(3))}
text = open(os.path.join(ref, "tests", "run", "mlp_mse.snap")).read().split("---")[-1]
out["mlp_mse"] = float(re.search(r"= ([-0-9.e]+)", text).group(1))
text = open(os.path.join(ref, "tests", "run", "mlp_mse_grad.snap")).read().split("---")[-1]
grad = {}
layer = None
for line in text.splitlines():
    m = re.match(r"\s*(l\d) = \{", line)
    if m:
        layer = m.group(1)
    m = re.match(r"\s*(w|b) = \[([0-9, ]+)\] (\[.*\])\s*$", line)
    if m:
        grad[layer + "." + m.group(1)] = {"shape": [int(x) for x in m.group(2).split(",")], "values": json.loads(m.group(3))}
out["mlp_mse_grad"] = grad
for name in ("rope_attention2", "rope_attention3"):
    text = open(os.path.join(ref, "tests", "run", name + ".snap")).read().split("---")[-1]
    m = re.search(r"\[batch: (\d+), seq: (\d+), model: (\d+)\] (\[\[\[.*\]\]\])", text)
    out[name] = {"shape": [int(m.group(1)), int(m.group(2)), int(m.group(3))], "values": json.loads(m.group(4))}
text = open(os.path.join(ref, "tests", "run", "concat_loss.snap")).read().split("---")[-1]
out["concat_loss"] = float(re.search(r"= ([-0-9.e]+)", text).group(1))
text = open(os.path.join(ref, "tests", "run", "concat_loss_grad.snap")).read().split("---")[-1]
grad = {}
for line in text.splitlines():
    m = re.match(r"\s*(tok|head|wq|wk|wv) = \[[a-z]+: (\d+), [a-z]+: (\d+)\] (\[\[.*\]\])\s*$", line)
    if m:
        path = m.group(1) if m.group(1) in ("tok", "head") else "qkv." + m.group(1)
        grad[path] = {"shape": [int(m.group(2)), int(m.group(3))], "values": json.loads(m.group(4))}
assert sorted(grad) == ["head", "qkv.wk", "qkv.wq", "qkv.wv", "tok"], sorted(grad)
out["concat_loss_grad"] = grad
text = open(os.path.join(ref, "tests", "run", "stack_grad.snap")).read().split("---")[-1]
grad = {}
for line in text.splitlines():
    m = re.match(r"\s*(w|b) = \[([0-9, ]+)\] (\[\[.*\]\])\s*$", line)
    if m:
        grad["blocks." + m.group(1)] = {"shape": [int(x) for x in m.group(2).split(",")], "values": json.loads(m.group(3))}
assert sorted(grad) == ["blocks.b", "blocks.w"], sorted(grad)
out["stack_grad"] = grad
key_rs = open(os.path.join(ref, "crates", "presk-interp", "src", "key.rs")).read()
m = re.search(r"assert_eq!\(first, \[([^\]]+)\]\)", key_rs)
out["seed0_first_normals_bits"] = [int(x.strip(), 16) for x in m.group(1).split(",")]
m = re.search(r"assert_eq!\(fold, (0x[0-9a-f]+)\)", key_rs)
out["seed0_next_100000_fnv"] = int(m.group(1), 16)
text = open(os.path.join(ref, "crates", "presk-kernel", "tests", "snapshots", "conformance__linear_kernels.snap")).read()
out["linear_kernels_text"] = text.split("---")[-1].lstrip("\n")
text = open(os.path.join(ref, "tests", "run", "minigpt_forward.snap")).read().split("---")[-1]
m = re.search(r"\[batch: (\d+), seq: (\d+), (\d+)\] (\[\[\[.*\]\]\])", text)
vals = json.loads(m.group(4))
flat = [x for b in vals for t in b for x in t]
out["minigpt_forward"] = {"shape": [int(m.group(1)), int(m.group(2)), int(m.group(3))], "all_equal_to": flat[0], "distinct": len(set(flat))}
text = open(os.path.join(ref, "tests", "run", "minigpt_loss.snap")).read().split("---")[-1]
out["minigpt_loss"] = float(re.search(r"= ([-0-9.e]+)", text).group(1))
with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json"), "w") as f:
    json.dump(out, f, indent=1)
print("wrote", list(out))

# The reference's own .psk.d files: their bytes, and what the header says (presk-data's layout: magic, u16 version,
# u32 length and text of the sample type, u64 count). The leaves are read off the type by hand.
import base64
import struct

files = {}
for rel, leaves in (("examples/tests/data/windows.psk.d", [(64, 8), (64, 8)]), ("examples/tests/train/reg.psk.d", [(0, 2), (0, 1)]),
                    ("examples/tutorial/data/pairs.psk.d", [(0, 4), (0, 4)]), ("examples/spec/minigpt/data/tokens.psk.d", [(64, 8), (64, 8)])):
    raw = open(os.path.join(ref, rel), "rb").read()
    assert raw[:4] == b"PSKD"
    version, tlen = struct.unpack("<HI", raw[4:10])
    typ = raw[10:10 + tlen].decode()
    count = struct.unpack("<Q", raw[10 + tlen:18 + tlen])[0]
    files[os.path.basename(rel)] = {"source": rel, "version": version, "type": typ, "count": count, "leaves": leaves, "bytes": base64.b64encode(raw).decode()}
with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "data_files.json"), "w") as f:
    json.dump(files, f, indent=0)
