"""Regenerate ``tests/golden/*.npz`` by running the REFERENCE implementation on CPU.

Usage (only where the reference checkout exists):
    python tests/golden/make_golden.py /path/to/reference

Inputs come from the bit-reproducible numpy generators in ``workloads.py`` so the
fixtures hold outputs only.  Every array written here was produced by the reference's own
``quantize`` / ``quantize_values`` / ``pack_pages`` / ``_reference_decode`` /
``InQuantCache`` code, not by this repository.
"""
from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "inquant-open-source_b200"))
sys.path.insert(0, HERE)
from cases import K4_CASES, V_CASES, PAGE_CASES, SELECT_CASES, DECODE_CASES, k4_input, select_input  # noqa: E402
import workloads  # noqa: E402


def main(ref_root: str) -> None:
    sys.modules["transformers"] = None  # reference cache falls back to its stub base class
    sys.path.insert(0, os.path.join(ref_root, "src"))
    sys.path.insert(0, os.path.join(ref_root, "extensions", "vllm", "src"))
    import torch
    from inquant.codec import CodecConfig, quantize, _reuse_map
    from inquant.value_codec import quantize_values
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.qwen_fused import _reference_decode
    from inquant_vllm.layout import PageLayout, pack_pages, unpack_pages_reference

    tdt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}

    def np_of(t):
        if t.dtype == torch.bfloat16:
            return t.float().numpy()
        return t.numpy()

    out = {}
    for name, case in K4_CASES.items():
        x = torch.from_numpy(k4_input(case)).to(tdt[case["dtype"]])
        packed = quantize(x, CodecConfig(sample_stride=case["stride"], salient_fraction=case["fraction"],
                                         donor_policy=case["policy"]))
        for field, tensor in packed.tensors.items():
            out[f"k4/{name}/{field}"] = np_of(tensor)
        deq = packed.dequantize().float().numpy()
        out[f"k4/{name}/dequant_sha256"] = np.frombuffer(hashlib.sha256(deq.tobytes()).digest(), np.uint8)
    for name, case in V_CASES.items():
        x = torch.from_numpy(k4_input(case)).to(tdt[case["dtype"]])
        packed = quantize_values(x, case["bits"], case["group"])
        for field, tensor in packed.tensors.items():
            out[f"v/{name}/{field}"] = np_of(tensor)
        deq = packed.dequantize().float().numpy()
        out[f"v/{name}/dequant_sha256"] = np.frombuffer(hashlib.sha256(deq.tobytes()).digest(), np.uint8)
    for name, case in SELECT_CASES.items():
        score, error = select_input(case)
        s, d = _reuse_map(torch.from_numpy(score), case["count"], None if error is None else torch.from_numpy(error))
        out[f"select/{name}/sources"] = s.numpy()
        out[f"select/{name}/donors"] = d.numpy()
    for name, case in PAGE_CASES.items():
        k, v = workloads.make_kv(case["seed"], case["heads"], case["pages"] * case["block"])
        shape = (case["heads"], case["pages"], case["block"], 128)
        kt = torch.from_numpy(k[0].reshape(shape).transpose(1, 0, 2, 3).copy()).bfloat16()
        vt = torch.from_numpy(v[0].reshape(shape).transpose(1, 0, 2, 3).copy()).bfloat16()
        layout = PageLayout(case["block"], case["heads"])
        pages = pack_pages(kt, vt, layout)
        out[f"pages/{name}/bytes"] = pages.numpy()
        rk, rv = unpack_pages_reference(pages, layout)
        out[f"pages/{name}/unpack_sha256"] = np.frombuffer(
            hashlib.sha256(rk.float().numpy().tobytes() + rv.float().numpy().tobytes()).digest(), np.uint8)
    for name, case in DECODE_CASES.items():
        k, v = workloads.make_kv(case["seed"], case["kv_heads"], case["tokens"], outliers=6, adjacent=3,
                                 scale_range=case["scale_range"])
        q = workloads.make_query(case["seed"], case["q_heads"])
        cfg = CacheConfig(CodecConfig(donor_policy="min_error"), block_size=case["block"],
                          residual_length=case["residual"], sink_tokens=case["sink"], value_bits=2,
                          value_group_size=64, validate_positions=False)
        cache = InQuantCache(cfg)
        kt, vt = torch.from_numpy(k).bfloat16(), torch.from_numpy(v).bfloat16()
        n = case["tokens"] - 1
        cache.update(kt[:, :, :n], vt[:, :, :n], 0)
        view = cache.append_for_attention(kt[:, :, n:], vt[:, :, n:], 0)
        qt = torch.from_numpy(q).bfloat16().view(1, case["q_heads"], 1, 128)
        result = _reference_decode(qt, view, 128 ** -0.5)
        out[f"decode/{name}/output"] = result.float().numpy().reshape(case["q_heads"], 128)
        out[f"decode/{name}/layout"] = np.array(
            [len(view.key_blocks), 0 if view.sink_key is None else view.sink_key.shape[2],
             view.residual_key.shape[2]], np.int64)
        digest = hashlib.sha256()
        for block in view.key_blocks:
            for field in ("payload", "scales", "salient_channels", "donor_channels", "padding"):
                digest.update(np_of(block.tensors[field]).tobytes())
        for block in view.value_blocks:
            for field in ("payload", "scales", "offsets"):
                digest.update(np_of(block.tensors[field]).tobytes())
        out[f"decode/{name}/packed_sha256"] = np.frombuffer(digest.digest(), np.uint8)
    np.savez_compressed(os.path.join(HERE, "reference_vectors.npz"), **out)
    print("wrote", len(out), "arrays,", os.path.getsize(os.path.join(HERE, "reference_vectors.npz")), "bytes")


if __name__ == "__main__":
    if len(sys.argv) < 2 and not os.environ.get("INQUANT_REFERENCE"):
        raise SystemExit("usage: make_golden.py <path of the reference checkout>  (or set INQUANT_REFERENCE)")
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ["INQUANT_REFERENCE"])
