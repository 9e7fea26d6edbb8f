"""The C++ decode layers (fastertransformer_b200/shim: DynamicDecodeLayer<T> with the reference's constructor,
setup() and forward() signatures and TensorMap keys) against the Python host mirror on the same seeded inputs.
Both sit on the same C ABI; the Python mirror is checked against the unmodified reference elsewhere, so equal
ids here show that the C++ host logic (argument broadcast, gating, slicing, stop criteria) is the same."""
import os
import subprocess

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRIVER = os.path.join(ROOT, "fastertransformer_b200", "lib", "shim_driver")
pytestmark = pytest.mark.gpu


def _mix(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)).astype(np.uint64)
    x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)).astype(np.uint64)
    return x ^ (x >> np.uint64(31))


def _unit(seed, n):
    with np.errstate(over="ignore"):
        m = _mix(np.uint64(seed) + np.arange(n, dtype=np.uint64))
    return ((m >> np.uint64(48)).astype(np.int64) - 32768).astype(np.float32) / np.float32(8192.0)


def _python_side(dtype, B, V, steps, which):
    from fastertransformer_b200 import DynamicDecodeLayer
    dev = torch.device("cuda:0")
    K = 4 if which == "beam" else 1
    mil, L = 4, 4 + steps
    idx = np.arange(B)
    if which == "topk":
        top_k, top_p = (1 + (idx * 5) % 40).astype(np.uint32), np.zeros(B, np.float32)
    elif which == "topp":
        top_k, top_p = np.zeros(B, np.uint32), (0.3 + 0.1 * (idx % 6)).astype(np.float32)
    else:
        top_k = np.asarray([0, 1, 8, 64], np.uint32)[idx % 4]
        top_p = np.asarray([0.0, 0.5, 0.9], np.float32)[(idx // 4) % 3]
    if K == 1:
        args = {"runtime_top_k": top_k, "runtime_top_p": top_p,
                "temperature": (0.5 + 0.25 * (idx % 4)).astype(np.float32),
                "repetition_penalty": np.asarray([1.2], np.float32),
                "random_seed": (100 + 7 * idx).astype(np.uint64)}
    else:
        args = {"len_penalty": np.asarray([1.0], np.float32)}
    layer = DynamicDecodeLayer(V, V, dtype, dev)
    layer.setup(B, K, args)
    ids = np.zeros((L, B * K), np.int32)
    with np.errstate(over="ignore"):
        for t in range(mil):
            ids[t] = (_mix(np.uint64(9000 + t * 131) + np.arange(B * K, dtype=np.uint64)) % np.uint64(V)).astype(np.int32)
    shape = (L, B) if K == 1 else (L, B, K)
    st = {"output_ids": torch.from_numpy(ids.reshape(shape)).to(dev),
          "finished": torch.zeros(B * K, dtype=torch.bool, device=dev),
          "sequence_length": torch.full((B * K,), mil, dtype=torch.int32, device=dev),
          "cum_log_probs": torch.from_numpy(-(np.arange(B * K) % K).astype(np.float32) if K > 1
                                            else np.zeros(B, np.float32)).to(dev)}
    if K > 1:
        st["parent_ids"] = torch.zeros(L, B, K, dtype=torch.int32, device=dev)
        st["tgt_cache_indirection"] = torch.zeros(B, K, L, dtype=torch.int32, device=dev)
    src = torch.zeros(B, K, L, dtype=torch.int32, device=dev)
    end = torch.full((B,), V - 1, dtype=torch.int32, device=dev)
    il = torch.full((B, K), mil, dtype=torch.int32, device=dev)
    lim = torch.full((B,), L, dtype=torch.int32, device=dev)
    lines = []
    for s in range(steps):
        step = mil + s
        x = torch.from_numpy(_unit(1000003 * (s + 1), B * K * V)).to(dev).to(dtype)
        inp = {"logits": x.view(B, V) if K == 1 else x.view(B, K, V), "step": step, "max_input_length": mil, "ite": 0,
               "local_batch_size": B, "end_id": end, "input_lengths": il, "sequence_limit_length": lim}
        if K > 1:
            inp.update(len_penalty=args["len_penalty"], src_cache_indirection=src)
        stop = layer.forward(st, inp)
        if K > 1:
            src, st["tgt_cache_indirection"] = st["tgt_cache_indirection"], src
        row = st["output_ids"][step].reshape(-1).cpu().numpy()
        lines.append("step %d stop %d ids %s" % (step, int(bool(stop)), " ".join(str(int(v)) for v in row)))
    return lines


CASES = [("f32", torch.float32, 6, 8, 6, "topk"), ("f32", torch.float32, 24, 2048, 4, "mixed"),
         ("f16", torch.float16, 24, 4096, 4, "topp"), ("bf16", torch.bfloat16, 36, 8192, 4, "mixed"),
         ("bf16", torch.bfloat16, 16, 8192, 3, "topk"), ("f16", torch.float16, 4, 4096, 4, "beam")]


@pytest.mark.parametrize("name,dtype,B,V,steps,which", CASES)
def test_cpp_layers_match_python_mirror(name, dtype, B, V, steps, which):
    if not os.path.exists(DRIVER):
        # built binaries normally travel with the tree; build here when this one did not
        from fastertransformer_b200.build import build_shim_driver
        build_shim_driver()
    assert os.path.exists(DRIVER), "shim driver not built: run python -m fastertransformer_b200.build"
    r = subprocess.run([DRIVER, name, str(B), str(V), str(steps), which], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    cpp = [l for l in r.stdout.strip().split("\n") if l.startswith("step")]
    py = _python_side(dtype, B, V, steps, which)
    assert cpp == py
