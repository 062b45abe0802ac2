#!/usr/bin/env python
"""Benchmark of the packed-KV hot path on B200.

Workload (N=1): Qwen2.5-7B-shaped single-request decode -- 28 layers x 4 KV heads x 128
head_dim, 28 query heads, 32768 history tokens packed K4/V2 (127 sealed blocks of 256 per
layer), bf16 attention sink (4) and recent tail (252, growing by one per step).  A "step"
is one decode step over ALL layers: the new token's K/V is appended to every layer's tail
and single-query GQA attention runs over every layer's packed history, sink and tail.
Inputs are seeded synthetic tensors with the reference workload's shapes and outlier
statistics (no model weights or datasets are used).

  python bench.py --gpus N --steps K --warmup W            this repository's CUDA path
  python bench.py --impl reference ...                     the CPU restatement of the reference
                                                           path, timed on the host cores

With N > 1 (torchrun, one rank per GPU) every rank serves its own request of the same shape
(requests shard across GPUs with no collective): weak scaling, value = sum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "inquant-open-source_b200"))

LAYERS, KV_HEADS, Q_HEADS, DIM = 28, 4, 28, 128
CONTEXT = 32768
BLOCK, RESIDUAL, SINK = 256, 128, 4
METRIC = "packed-KV decode attn HBM GB/s at 32K ctx (all 28 layers per step)"


def blocks_bytes_encode():
    """Algorithmic bytes of sealing one layer: bf16 K and V read, packed fields written."""
    blocks = (CONTEXT - SINK - RESIDUAL) // BLOCK
    per_token_head = 2 * DIM * 2 + 64 + 32 + 8
    return blocks * KV_HEADS * (BLOCK * per_token_head + 512 + 16 + 16 + 64)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML (read-only queries) from a
    background thread while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz, self._stop, self._thread, self._nvml = None, threading.Event(), None, None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._nvml = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        except Exception:
            self._nvml = None
        return self

    def _run(self):
        nv = self._nvml
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(self.period)

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self):
        clocks = sorted(self.samples)
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(clocks)}



# --------------------------------------------------------------------------- parity against the oracle
# Every timed leg is followed, outside its timed region, by a comparison of a sample of the
# outputs it produced with the CPU oracle (the checker, never the thing measured): attention
# within max-abs 2e-2 and cosine >= 0.9999, packed bytes and descriptors bit for bit.  A failed
# comparison ends the run with a non-zero exit code.
PARITY_MAX_ABS, PARITY_MIN_COS = 2e-2, 0.9999


class ParityError(SystemExit):
    def __init__(self, what):
        super().__init__(f"parity check failed: {what}")


def _oracle():
    path = os.path.join(ROOT, "oracle")
    if path not in sys.path:
        sys.path.insert(0, path)
    import inquant_oracle
    return inquant_oracle


def _closeness(got, want):
    import numpy as np
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = float(np.abs(got - want).max())
    cos = (got * want).sum(-1) / np.sqrt((got * got).sum(-1) * (want * want).sum(-1) + 1e-300)
    return err, float(cos.min()), bool(np.isfinite(got).all())


def _host(t):
    import torch
    t = t.detach()
    return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()


def oracle_packed(oracle, key_blocks, value_blocks):
    """The device's packed blocks (lists of [1, H, T, ...] fields) as the oracle's containers."""
    import torch
    cat = lambda blocks, name: _host(torch.cat([getattr(b, name) for b in blocks], 0))
    n, heads, tokens = len(key_blocks), key_blocks[0].payload.shape[1], key_blocks[0].payload.shape[2]
    shape = (n, heads, tokens, DIM)
    pk = oracle.PackedK(cat(key_blocks, "payload"), cat(key_blocks, "scales"), cat(key_blocks, "salient_channels"),
                        cat(key_blocks, "donor_channels"), cat(key_blocks, "padding"), shape, "bfloat16")
    pv = oracle.PackedV(cat(value_blocks, "payload"), scales=cat(value_blocks, "scales"), offsets=cat(value_blocks, "offsets"),
                        shape=shape, dtype="bfloat16", bits=2, group_size=64)
    return pk, pv


def oracle_dense_history(oracle, pk, pv, sink, tail):
    """[H, tokens, 128] keys and values the reference's oracle attends to: exact sink, dequantised
    blocks rounded to bf16, exact tail."""
    import numpy as np
    heads = pk.shape[1]
    keys = oracle.dequantize_k4(pk).transpose(1, 0, 2, 3).reshape(heads, -1, DIM)
    vals = oracle.dequantize_values(pv).transpose(1, 0, 2, 3).reshape(heads, -1, DIM)
    return (np.concatenate([sink[0], keys, tail[0]], 1), np.concatenate([sink[1], vals, tail[1]], 1))


def layer_dense_parts(cache, layer_idx, tail_tokens):
    layer = cache._layers[layer_idx]
    sink = (_host(layer.sink_key)[0], _host(layer.sink_value)[0])
    tail = (_host(layer.tail_key_buffer[:, :, :tail_tokens])[0], _host(layer.tail_value_buffer[:, :, :tail_tokens])[0])
    return sink, tail


def check_decode_parity(torch, batch, cache, layers, seed_base, encode_layer=0):
    """Config 1 at full size: the outputs of the 28-layer launch for `layers` against the oracle's
    attention over the device's own packed bytes, and the packed fields of one whole layer
    (127 blocks x 4 heads) bit for bit against the oracle's encoders on the same seeded tensors."""
    import numpy as np
    import workloads
    oracle = _oracle()
    torch.cuda.synchronize()
    outputs = _host(batch.outputs)
    queries = _host(batch.queries)
    tails = batch.tail_tokens
    worst, lowest = 0.0, 1.0
    for index in layers:
        state = batch.sequences[index].decode_state
        pk, pv = oracle_packed(oracle, state.key_blocks, state.value_blocks)
        sink, tail = layer_dense_parts(cache, index, tails[index])
        keys, vals = oracle_dense_history(oracle, pk, pv, sink, tail)
        want = oracle.attention_decode(queries[index], keys, vals, DIM ** -0.5)
        err, cos, finite = _closeness(outputs[index], want)
        worst, lowest = max(worst, err), min(lowest, cos)
        if not finite or err >= PARITY_MAX_ABS or cos < PARITY_MIN_COS:
            raise ParityError(f"config 1 decode, layer {index}: max abs {err:.3e}, min cosine {cos:.6f}")
    # one layer's packed bytes and descriptors against the oracle's encoders
    k, v = workloads.make_kv_torch(seed_base + encode_layer, KV_HEADS, CONTEXT, batch.device)
    take, blocks, _ = oracle.seal_plan(0, 0, CONTEXT, sink_tokens=SINK, residual_length=RESIDUAL, block_size=BLOCK)
    body = slice(take, take + blocks * BLOCK)
    shape = (KV_HEADS, blocks, BLOCK, DIM)
    kb = np.ascontiguousarray(_host(k)[0][:, body].reshape(shape).transpose(1, 0, 2, 3))
    vb = np.ascontiguousarray(_host(v)[0][:, body].reshape(shape).transpose(1, 0, 2, 3))
    del k, v
    want_k = oracle.quantize_k4(kb, "bfloat16", 8, 0.125, "min_error")
    want_v = oracle.quantize_values(vb, "bfloat16", 2, 64)
    state = batch.sequences[encode_layer].decode_state
    got_k, got_v = oracle_packed(oracle, state.key_blocks, state.value_blocks)
    mismatches = 0
    for got, want in ((got_k, want_k), (got_v, want_v)):
        for name, array in want.fields().items():
            have = getattr(got, name)
            if have.shape != array.shape or have.dtype != array.dtype:
                raise ParityError(f"config 1 encode, field {name}: {have.dtype}{have.shape} vs {array.dtype}{array.shape}")
            mismatches += int(np.count_nonzero(np.ascontiguousarray(have).view(np.uint8) != np.ascontiguousarray(array).view(np.uint8)))
    if mismatches:
        raise ParityError(f"config 1 encode, layer {encode_layer}: {mismatches} packed bytes differ from the oracle")
    return {"max_abs": round(worst, 6), "min_cos": round(lowest, 7), "layers_checked": list(layers),
            "against": "oracle f64 attention over the device's packed bytes (exact sink and tail), all layers in one launch",
            "encode_layer_checked": encode_layer, "encode_blocks_checked": blocks * KV_HEADS,
            "encode_mismatched_bytes": mismatches}


def check_split_parity(torch, dist, split, cache, run_step, step_inputs, world, rank, first, last, layer=0):
    """Config 4: the merged output of one layer against the oracle's attention over the WHOLE
    request.  Every rank computes the oracle's partial record (acc, m, l) over its own shard of
    the history from the device's packed bytes; the records are gathered and merged as the
    reference's reduce kernel merges them (at one rank that is the unsplit oracle)."""
    import numpy as np
    oracle = _oracle()
    split.inputs.copy_(step_inputs)
    run_step()
    torch.cuda.synchronize()
    batch = split.batch
    state = batch.sequences[layer].decode_state
    pk, pv = oracle_packed(oracle, state.key_blocks, state.value_blocks)
    heads = pk.shape[1]
    cache_layer = cache._layers[layer]
    empty = np.zeros((heads, 0, DIM), np.float32)
    sink = (_host(cache_layer.sink_key)[0], _host(cache_layer.sink_value)[0]) if first and cache_layer.sink_key is not None else (empty, empty)
    tail_tokens = batch.tail_tokens[layer] if last else 0
    tail = ((_host(cache_layer.tail_key_buffer[:, :, :tail_tokens])[0], _host(cache_layer.tail_value_buffer[:, :, :tail_tokens])[0])
            if tail_tokens else (empty, empty))
    keys, vals = oracle_dense_history(oracle, pk, pv, sink, tail)
    query = _host(batch.queries)[layer]
    record = oracle.attention_partial(query, keys, vals, DIM ** -0.5)
    records = [record]
    if world > 1:
        records = [None] * world
        dist.all_gather_object(records, record)
    acc, m, l = (np.stack([r[i] for r in records]) for i in range(3))
    want = oracle.merge_partials(acc, m, l)
    err, cos, finite = _closeness(_host(split.outputs)[layer], want)
    if not finite or err >= PARITY_MAX_ABS or cos < PARITY_MIN_COS:
        raise ParityError(f"config 4 split-KV, layer {layer}, rank {rank}: max abs {err:.3e}, min cosine {cos:.6f}")
    return {"max_abs": round(err, 6), "min_cos": round(cos, 7), "layers_checked": [layer],
            "against": "oracle partial records of every rank's shard, merged; equal to the unsplit oracle"}


def check_paged_parity(torch, batch, seqs, local_lengths, layers, block, heads, layer=1):
    """Config 3: the shortest and the longest request of this rank, one layer each, against the
    oracle: the pages' bytes are unpacked as the reference's `unpack_pages_reference` does, the
    exact sink replaces the first packed tokens, the exact tail follows."""
    import numpy as np
    oracle = _oracle()
    torch.cuda.synchronize()
    outputs, queries = _host(batch.outputs), _host(batch.queries)
    order = sorted(range(len(local_lengths)), key=lambda i: local_lengths[i])
    picks = sorted({order[0], order[-1]})
    worst, lowest = 0.0, 1.0
    for pick in picks:
        index = pick * layers + min(layer, layers - 1)
        seq = seqs[index]
        pages = seq.pool[seq.page_table.long()].cpu().numpy()
        keys, vals = oracle.unpack_pages(pages, block, heads)
        keys = keys.transpose(1, 0, 2, 3).reshape(heads, -1, DIM).copy()
        vals = vals.transpose(1, 0, 2, 3).reshape(heads, -1, DIM).copy()
        dense = _host(seq.dense)
        sink, tail = seq.sink_count, seq.tail_count
        keys[:, :sink], vals[:, :sink] = dense[0][:, :sink], dense[1][:, :sink]
        keys = np.concatenate([keys, dense[0][:, 4:4 + tail]], 1)
        vals = np.concatenate([vals, dense[1][:, 4:4 + tail]], 1)
        want = oracle.attention_decode(queries[index], keys, vals, DIM ** -0.5)
        err, cos, finite = _closeness(outputs[index], want)
        worst, lowest = max(worst, err), min(lowest, cos)
        if not finite or err >= PARITY_MAX_ABS or cos < PARITY_MIN_COS:
            raise ParityError(f"config 3 paged decode, block {block}, request of {local_lengths[pick]} tokens: "
                              f"max abs {err:.3e}, min cosine {cos:.6f}")
    return {"max_abs": round(worst, 6), "min_cos": round(lowest, 7),
            "requests_checked": [int(local_lengths[i]) for i in picks], "layer": min(layer, layers - 1),
            "against": "oracle f64 attention over the unpacked page bytes (exact sink and tail)"}


# --------------------------------------------------------------------------- CUDA arm
def build_request(torch, device, seed_base):
    """Prefill all layers through the public cache API; returns the cache and encode timings."""
    import workloads
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error", donor_backend="triton"), block_size=BLOCK,
                                     residual_length=RESIDUAL, sink_tokens=SINK, value_bits=2, value_group_size=64,
                                     validate_positions=False))
    encode_ms = 0.0
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for layer in range(LAYERS):
        k, v = workloads.make_kv_torch(seed_base + layer, KV_HEADS, CONTEXT, device)
        # a throw-away prefill of the same tensors first: it warms the kernels and leaves its
        # device blocks in torch's caching allocator, so the timed prefill measures the encoders
        # and the cache bookkeeping, not cudaMalloc (a serving engine seals into a preallocated pool)
        warm = InQuantCache(cache.config)
        warm.update(k, v, 0)
        del warm
        torch.cuda.synchronize()
        start.record()
        cache.update(k, v, layer)
        stop.record()
        torch.cuda.synchronize()
        encode_ms += start.elapsed_time(stop)
        if layer == LAYERS - 1:
            kernels_us = encoder_kernels_us(torch, k, v)
        del k, v
    return cache, encode_ms, kernels_us


def measure_append_and_seal(torch, batch, device):
    """The append kernel alone (one launch writes the new token of all 28 layers into tail, and
    sink while it fills) and the sealing of one 256-token block of one layer (K4 + V2 encoders on
    [1, 4, 256, 128], including the finite-check read-back) through the cache and through the two
    codec calls: a block is sealed once per 256 decoded tokens and layer."""
    from inquant.codec import CodecConfig, quantize
    from inquant.value_codec import quantize_values
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    batch.rewind()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        batch._launch_append()
    e1.record()
    torch.cuda.synchronize()
    append_us = e0.elapsed_time(e1) / reps * 1e3
    batch.rewind()
    gen = torch.Generator(device=device).manual_seed(5)
    block_k = torch.randn((1, KV_HEADS, BLOCK, DIM), device=device, generator=gen).bfloat16()
    block_v = torch.randn((1, KV_HEADS, BLOCK, DIM), device=device, generator=gen).bfloat16()
    cfg = CodecConfig(donor_policy="min_error", donor_backend="triton")
    for _ in range(3):
        quantize(block_k, cfg), quantize_values(block_v, 2, 64)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        quantize(block_k, cfg), quantize_values(block_v, 2, 64)
    e1.record()
    torch.cuda.synchronize()
    codec_us = e0.elapsed_time(e1) / reps * 1e3
    # the same block sealed the way the cache does it: one `extend` (`update` without the dense history it returns) of BLOCK tokens on a layer whose
    # tail is full seals exactly one block (both encoders and the tail copy from one host call, one
    # read of the status word)
    from inquant.cache import CacheConfig, InQuantCache
    cache = InQuantCache(CacheConfig(cfg, block_size=BLOCK, residual_length=RESIDUAL, sink_tokens=SINK, value_bits=2,
                                     value_group_size=64, validate_positions=False))
    first = torch.randn((1, KV_HEADS, SINK + RESIDUAL, DIM), device=device, generator=gen).bfloat16()
    cache.extend(first, first, 0)
    for _ in range(3):
        cache.extend(block_k, block_v, 0)
    torch.cuda.synchronize()
    before = len(cache._layers[0].key_blocks)
    # one event per repetition and the median of the intervals: every seal keeps its block's tensors,
    # so now and then torch's allocator goes to cudaMalloc for a new segment, which says nothing
    # about the sealing path (the worst interval is reported beside the median)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    marks[0].record()
    for i in range(reps):
        cache.extend(block_k, block_v, 0)
        marks[i + 1].record()
    torch.cuda.synchronize()
    assert len(cache._layers[0].key_blocks) == before + reps
    intervals = sorted(marks[i].elapsed_time(marks[i + 1]) * 1e3 for i in range(reps))
    seal_us = intervals[reps // 2]
    return {"append_us_all_layers": round(append_us, 2), "seal_us_per_block_and_layer": round(seal_us, 1),
            "seal_us_per_token_amortised_all_layers": round(seal_us * LAYERS / BLOCK, 2),
            "seal_us_worst_of_%d" % reps: round(intervals[-1], 1),
            "codec_calls_us_per_block": round(codec_us, 1),
            "what": "seal: InQuantCache.extend of one 256-token chunk on one layer (K4 + V2 encoders, tail copy, "
                    "finite-check read-back), median of the repetitions; codec_calls: quantize + quantize_values of the same block, each with its own read-back"}


def encoder_kernels_us(torch, k, v):
    """Device time of the two encoder launches that seal one layer (127 blocks x 4 heads of keys,
    then of values), launched back to back into preallocated outputs through the C ABI without
    the finite-check read-back: the encoders alone, without cache bookkeeping."""
    from inquant import _native as N
    from inquant.codec import CodecConfig, encode_into
    from inquant.value_codec import encode_values_into
    blocks = (CONTEXT - SINK - RESIDUAL) // BLOCK
    device = k.device
    kb = k[0, :, SINK:SINK + blocks * BLOCK].reshape(KV_HEADS, blocks, BLOCK, DIM).permute(1, 0, 2, 3)
    vb = v[0, :, SINK:SINK + blocks * BLOCK].reshape(KV_HEADS, blocks, BLOCK, DIM).permute(1, 0, 2, 3)
    cfg = CodecConfig(donor_policy="min_error", donor_backend="triton")
    count = DIM // 8
    payload = torch.empty((blocks, KV_HEADS, BLOCK, DIM // 2), dtype=torch.uint8, device=device)
    scales = torch.empty((blocks, KV_HEADS, DIM), dtype=torch.float32, device=device)
    salient = torch.empty((blocks, KV_HEADS, count), dtype=torch.uint8, device=device)
    donors = torch.empty_like(salient)
    padding = torch.empty((blocks, KV_HEADS, count), dtype=torch.float32, device=device)
    vpayload = torch.empty((blocks, KV_HEADS, BLOCK, DIM // 4), dtype=torch.uint8, device=device)
    vscales = torch.empty((blocks, KV_HEADS, BLOCK, 2), dtype=torch.float16, device=device)
    voffsets = torch.empty_like(vscales)
    f = lambda t: N.compact_field(t, KV_HEADS)

    def once():
        encode_into(kb, cfg, f(payload), f(scales), f(salient), f(donors), f(padding))
        encode_values_into(vb, 2, 64, f(vpayload), f(vscales), f(voffsets))
    for _ in range(3):
        once()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        once()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / 10 * 1e3


def value_codecs_leg(torch, device):
    """One layer of config 1 under every value codec the one-launch kernel serves: the preset (2-bit,
    groups of 64), values stored as InQuant packed tensors (the reference's `CacheConfig` default),
    4-bit values in groups of 64 and 32, 2-bit values in groups of 128 and 32.  Ten decodes per CUDA-graph
    replay, device time per launch; each output is compared with the general kernel's for the same state
    (the tests hold both against the oracle)."""
    import workloads
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.triton_attention import PackedDecodeState
    k, v = workloads.make_kv_torch(77, KV_HEADS, CONTEXT, device)
    gen = torch.Generator(device=device).manual_seed(78)
    q = torch.randn((1, Q_HEADS, 1, DIM), device=device, generator=gen).bfloat16()
    out = {}
    codecs = (("k4_v2_g64", dict(value_bits=2, value_group_size=64)), ("k4_values_as_inquant_tensors", dict(value_bits=None)),
              ("k4_v4_g64", dict(value_bits=4, value_group_size=64)), ("k4_v4_g32", dict(value_bits=4, value_group_size=32)),
              ("k4_v2_g128", dict(value_bits=2, value_group_size=128)), ("k4_v2_g32", dict(value_bits=2, value_group_size=32)))
    for name, kw in codecs:
        cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=BLOCK, residual_length=RESIDUAL,
                                         sink_tokens=SINK, validate_positions=False, **kw))
        cache.update(k, v, 0)
        layer = cache._layers[0]
        dense = dict(sink_key=layer.sink_key, sink_value=layer.sink_value, residual_key=layer.residual_key,
                     residual_value=layer.residual_value)
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            state = PackedDecodeState(layer.key_blocks, layer.value_blocks)
            for _ in range(3):
                result = state.decode(q, **dense)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(10):
                    result = state.decode(q, **dense)
            graph.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(5):
                graph.replay()
            e1.record(side)
            side.synchronize()
            general = state._decode_general(q, KV_HEADS, Q_HEADS // KV_HEADS, len(layer.key_blocks), layer.sink_key, layer.sink_value,
                                            layer.sink_key.shape[2], layer.residual_key, layer.residual_value,
                                            layer.residual_key.shape[2], DIM ** -0.5)
            side.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 50
        nbytes = sum(b.nbytes for b in layer.key_blocks) + sum(b.nbytes for b in layer.value_blocks)
        diff = float((result.float() - general.float()).abs().max())
        if not diff < PARITY_MAX_ABS:
            raise ParityError(f"value codec {name}: one-launch kernel and general kernel differ by {diff:.3e}")
        out[name] = {"us_per_layer": round(us, 2), "packed_mb": round(nbytes / 1e6, 2), "packed_gbs": round(nbytes / us / 1e3, 1),
                     "streaming_value_kind": list(state.streaming_value_kind()), "max_abs_vs_general_kernel": round(diff, 6)}
        del cache, state, graph
    out["note"] = ("one layer (14-19 MB) stays in the 126 MB L2 between the replays: these are L2-warm times, to be compared "
                   "with one another and with reference_gpu.warm, not with the 28-layer figures")
    return out


def reference_gpu_leg(torch, device):
    """One layer of config 1 through the UNMODIFIED reference on this GPU (installed under
    oracle/_ref): its torch CUDA encoders against this library's encoders byte by byte, and its
    Triton decode kernels (`PackedDecodeState.decode`: partials + reduce) timed in alternation with
    this library's single-layer decode on the same packed layer, warm and with L2 flushed."""
    import importlib
    import workloads
    ref = _reference_modules()
    if ref is None:
        return {"unavailable": "oracle/_ref is missing (the reference checkout was absent when the library was built)"}
    try:
        rta = importlib.import_module("inquant_reference.triton_attention")
    except Exception as exc:
        return {"unavailable": f"the reference's Triton module did not import: {exc}"}
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.triton_attention import PackedDecodeState
    k, v = workloads.make_kv_torch(424242, KV_HEADS, CONTEXT, device)
    rcodec, rcache = ref["codec"], ref["cache"]
    theirs = rcache.InQuantCache(rcache.CacheConfig(rcodec.CodecConfig(donor_policy="min_error", donor_backend="torch"),
                                                    block_size=BLOCK, residual_length=RESIDUAL, sink_tokens=SINK, value_bits=2,
                                                    value_group_size=64, validate_positions=False))
    ours = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=BLOCK, residual_length=RESIDUAL,
                                    sink_tokens=SINK, value_bits=2, value_group_size=64, validate_positions=False))
    theirs.update(k, v, 0)
    ours.update(k, v, 0)
    a, b = theirs._layers[0], ours._layers[0]
    mismatch, total = {}, 0
    for kind, fields in (("key", ("payload", "scales", "salient_channels", "donor_channels", "padding")),
                         ("value", ("payload", "scales", "offsets"))):
        for name in fields:
            x = torch.cat([getattr(blk, name) for blk in getattr(a, kind + "_blocks")], 0).contiguous().view(torch.uint8)
            y = torch.cat([getattr(blk, name) for blk in getattr(b, kind + "_blocks")], 0).contiguous().view(torch.uint8)
            count = int((x != y).sum().item()) if x.shape == y.shape else -1
            mismatch[f"{kind}_{name}"] = count
            total += max(count, 0)
    gen = torch.Generator(device=device).manual_seed(11)
    new_k = torch.randn((1, KV_HEADS, 1, DIM), device=device, generator=gen).bfloat16()
    new_v = torch.randn((1, KV_HEADS, 1, DIM), device=device, generator=gen).bfloat16()
    q = torch.randn((1, Q_HEADS, 1, DIM), device=device, generator=gen).bfloat16()
    view_a = theirs.append_for_attention(new_k, new_v, 0)
    view_b = ours.append_for_attention(new_k, new_v, 0)
    state_a = rta.PackedDecodeState(list(view_a.key_blocks), list(view_a.value_blocks))
    state_b = PackedDecodeState(view_b.key_blocks, view_b.value_blocks)
    dense_a = dict(sink_key=view_a.sink_key, sink_value=view_a.sink_value, residual_key=view_a.residual_key, residual_value=view_a.residual_value)
    dense_b = dict(sink_key=view_b.sink_key, sink_value=view_b.sink_value, residual_key=view_b.residual_key, residual_value=view_b.residual_value)
    out_a = state_a.decode(q, **dense_a)
    out_b = state_b.decode(q, **dense_b)
    torch.cuda.synchronize()
    diff = float((out_a.float() - out_b.float()).abs().max().item())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    # Both decodes are captured in CUDA graphs where the capture succeeds, so that the events time
    # the kernels and not the Python around them (the reference's call spends more host time than
    # device time); otherwise the calls are timed eagerly and the record says so.
    def graphed(make_state, dense):
        # state, warm-up and capture all on ONE side stream (both libraries tie a state to its stream)
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                state = make_state()
                state.decode(q, **dense)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                state.decode(q, **dense)
            graph.replay()
            torch.cuda.synchronize()
            return graph.replay, "CUDA graph replay", state
        except Exception as exc:
            torch.cuda.synchronize()
            state = make_state()
            return (lambda: state.decode(q, **dense)), f"eager call (capture failed: {type(exc).__name__}: {exc})"[:160], state
    run_a, how_a, keep_a = graphed(lambda: rta.PackedDecodeState(list(view_a.key_blocks), list(view_a.value_blocks)), dense_a)
    run_b, how_b, keep_b = graphed(lambda: PackedDecodeState(view_b.key_blocks, view_b.value_blocks), dense_b)
    result = {"timed_as": {"reference_triton": how_a, "this_library": how_b}}
    for label, do_flush in (("warm", False), ("l2_flushed", True)):
        times_a, times_b = [], []
        for _ in range(30):   # alternate the two kernels so both see the same clocks
            for run, bucket in ((run_a, times_a), (run_b, times_b)):
                if do_flush:
                    flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                run()
                e1.record()
                torch.cuda.synchronize()
                bucket.append(e0.elapsed_time(e1) * 1e3)
        result[label] = {"reference_triton_us": round(sorted(times_a)[len(times_a) // 2], 2),
                         "this_library_us": round(sorted(times_b)[len(times_b) // 2], 2)}
    blocks, tail = len(view_b.key_blocks), view_b.residual_key.shape[2]
    return {"workload": "config 1, ONE layer (32768 tokens, 4 KV heads, 28 query heads), single-layer launches timed in alternation",
            "reference": "unmodified reference from oracle/_ref: torch CUDA encoders (donor_backend=torch), Triton partials + reduce kernels",
            "encoder_bytes_differing_from_reference_cuda": mismatch, "encoder_bytes_differing_total": total,
            "decode_max_abs_diff_vs_reference_triton": round(diff, 5), "layer_bytes": layer_bytes(blocks, tail), **result}


def append_sequence_leg(torch, device, cache, steps=136):
    """Config 1's incremental appends on ONE cache through the public per-layer API: every step
    appends one token to all 28 layers (`append_for_attention`) and attends (`PackedDecodeState.decode`).
    From a 32768-token prefill the tail holds 252 tokens, so 131 appends fit the tail and append 132
    seals a block in every layer (reference `cache.py:271-306`); the run crosses that seal and ends
    with a comparison of one layer's output, new block included, with the oracle."""
    import numpy as np
    from inquant.triton_attention import PackedDecodeState, SharedDecodeWorkspace
    oracle = _oracle()
    layers = sorted(cache._layers)
    pool = SharedDecodeWorkspace()
    states = [PackedDecodeState(cache._layers[i].key_blocks, cache._layers[i].value_blocks, workspace_pool=pool) for i in layers]
    blocks_before = len(states[0].key_blocks)
    gen = torch.Generator(device=device).manual_seed(2718)
    feed = torch.randn((steps, len(layers), Q_HEADS + 2 * KV_HEADS, DIM), device=device, generator=gen).bfloat16()
    times, seal_steps = [], []
    out = view = None
    for step in range(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for slot, index in enumerate(layers):
            row = feed[step, slot]
            q = row[:Q_HEADS].view(1, Q_HEADS, 1, DIM)
            new_k = row[Q_HEADS:Q_HEADS + KV_HEADS].view(1, KV_HEADS, 1, DIM)
            new_v = row[Q_HEADS + KV_HEADS:].view(1, KV_HEADS, 1, DIM)
            view = cache.append_for_attention(new_k, new_v, index)
            if len(view.key_blocks) != len(states[slot].key_blocks):
                states[slot].extend(view.key_blocks, view.value_blocks)
            out = states[slot].decode(q, sink_key=view.sink_key, sink_value=view.sink_value,
                                      residual_key=view.residual_key, residual_value=view.residual_value)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
        if len(cache._layers[layers[0]].key_blocks) != blocks_before + len(seal_steps):
            seal_steps.append(step + 1)
    # the last layer's last output against the oracle (its view holds the block sealed on the way)
    pk, pv = oracle_packed(oracle, list(view.key_blocks), list(view.value_blocks))
    sink = (_host(view.sink_key)[0], _host(view.sink_value)[0])
    tail = (_host(view.residual_key)[0], _host(view.residual_value)[0])
    keys, vals = oracle_dense_history(oracle, pk, pv, sink, tail)
    want = oracle.attention_decode(_host(feed[steps - 1, len(layers) - 1, :Q_HEADS]), keys, vals, DIM ** -0.5)
    err, cos, finite = _closeness(_host(out).reshape(Q_HEADS, DIM), want)
    if not finite or err >= PARITY_MAX_ABS or cos < PARITY_MIN_COS:
        raise ParityError(f"config 1 append sequence, last step: max abs {err:.3e}, min cosine {cos:.6f}")
    plain = [t for i, t in enumerate(times) if i + 1 not in seal_steps and i >= 3]
    return {"what": "per-layer public API: append_for_attention + PackedDecodeState.decode for each of the layers, one token per step",
            "steps": steps, "us_per_step_median_without_seal": round(float(np.median(plain)), 1),
            "first_128_steps_ms": round(sum(times[:128]) / 1e3, 3),
            "seal_at_append": seal_steps, "us_of_sealing_steps": [round(times[i - 1], 1) for i in seal_steps],
            "blocks_per_layer_before_after": [blocks_before, len(cache._layers[layers[0]].key_blocks)],
            "parity_last_step": {"max_abs": round(err, 6), "min_cos": round(cos, 7), "blocks": len(view.key_blocks)}}


def sustained_leg(torch, batch, run_step, device_index, seconds):
    """The same step replayed back to back for `seconds` of device time: on this pool the SM clock
    settles well below its boost value under seconds of load, and a kernel that is bound by
    latency or issue rate slows down with it.  Clocks are sampled, never set."""
    chunk = max(1, min(100, batch._capacity - 1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = 0
    with ClockSampler(device_index, period_s=0.005) as clocks:
        wall = time.perf_counter()
        e0.record()
        while time.perf_counter() - wall < seconds:
            batch.rewind()
            for _ in range(chunk):
                run_step()
            steps += chunk
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / steps
    summary = clocks.summary()
    return {"what": "the same decode step replayed back to back; tails rewound every %d steps (one small copy)" % chunk,
            "seconds": round(e0.elapsed_time(e1) / 1e3, 2), "steps": steps, "us_per_step": round(us, 2),
            "sm_mhz_median": summary["sm_mhz"], "sm_max_mhz": summary["sm_max_mhz"], "clock_samples": summary["samples"],
            "reasons": summary["reasons"],
            "us_times_mhz": round(us * summary["sm_mhz"], 0) if summary["sm_mhz"] else None}


def run_cuda(args):
    import torch
    import torch.distributed as dist
    from inquant import _native
    from inquant.batched import DecodeBatch, SequenceState

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the packed-KV path has no CPU fallback")
    _native.library()
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    cache, encode_ms, encode_kernels_us = build_request(torch, device, seed_base=1000 * rank)
    batch = DecodeBatch([SequenceState.from_cache_layer(cache, i) for i in range(LAYERS)], Q_HEADS, torch.bfloat16)
    total_steps = args.warmup + args.steps
    gen = torch.Generator(device=device).manual_seed(7 + rank)
    # per step and layer: 28 query heads, then the new token's 4 key heads and 4 value heads
    inputs = torch.randn((total_steps, LAYERS, Q_HEADS + 2 * KV_HEADS, DIM), device=device, generator=gen).bfloat16()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (inputs already in HBM): per step one staging copy, then the
    # CUDA graph of {append kernel, decode kernel}
    for i in range(args.warmup):
        batch.inputs.copy_(inputs[i])
        batch.step()
    torch.cuda.synchronize()
    use_graph = not args.no_graph
    if use_graph:
        batch.capture()
    run_step = batch.replay if use_graph else batch.step
    for i in range(args.warmup):
        if batch.capacity_left < 1:
            batch.rewind()
        batch.inputs.copy_(inputs[i])
        run_step()
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    byte_samples = []
    launches_before = batch.launches
    with ClockSampler(local) as clocks:
        t0.record()
        for i in range(args.steps):
            if batch.capacity_left < 1:
                batch.rewind()
            batch.inputs.copy_(inputs[args.warmup + i])
            run_step()
            byte_samples.append(batch._appended)
        t1.record()
        barrier()
        # ---- the decode kernel alone, back to back, for the roofline figure
        reps = max(args.steps, 20)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            batch.attend()
        torch.cuda.synchronize()
        k0.record()
        for _ in range(reps):
            batch._launch_attend()
        k1.record()
        torch.cuda.synchronize()
    elapsed_ms = t0.elapsed_time(t1)
    launches = batch.launches - launches_before - 3
    sustained = sustained_leg(torch, batch, run_step, local, args.sustained_seconds) if args.sustained_seconds > 0 else None
    kernel_ms = k0.elapsed_time(k1) / reps
    append_info = measure_append_and_seal(torch, batch, device)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    base = batch.algorithmic_bytes()
    per_token = KV_HEADS * DIM * 2 * 2 * LAYERS
    mean_appended = sum(byte_samples) / len(byte_samples) - batch._appended
    mean_bytes = dict(base)
    mean_bytes["dense"] = base["dense"] + mean_appended * per_token
    mean_bytes["total"] = base["total"] + mean_appended * per_token
    kernel_bytes = base["total"]
    ms_per_step = elapsed_ms / args.steps
    value = world * mean_bytes["total"] / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through the public API with host buffers
    if args.skip_e2e:
        if rank == 0:
            print(json.dumps({"layers": LAYERS, "us_per_step": round(ms_per_step * 1e3, 2),
                              "decode_us_per_launch": round(kernel_ms * 1e3, 2), "kernel_bytes": kernel_bytes,
                              "encode_ms": round(encode_ms, 3)}))
        return
    batch.rewind()
    h_in = inputs.cpu().pin_memory()
    h_out = torch.empty((LAYERS, Q_HEADS, DIM), dtype=torch.bfloat16).pin_memory()

    def host_step(i):
        if batch.capacity_left < 1:
            batch.rewind()
        batch.inputs.copy_(h_in[i], non_blocking=True)
        out = run_step()
        h_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the next token depends on this result

    for i in range(args.warmup):
        host_step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        host_step(args.warmup + i)
    e1.record()
    barrier()
    e2e_ms = max(e0.elapsed_time(e1), (time.perf_counter() - wall0) * 1e3) / args.steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = h_in[0].numel() * 2
    d2h = h_out.numel() * 2
    status = _native.take_status(device)
    # ---- parity of what was just timed (outside every timed region)
    batch.rewind()
    batch.inputs.copy_(inputs[0])
    run_step()
    parity = check_decode_parity(torch, batch, cache, sorted({0, LAYERS // 2, LAYERS - 1}), seed_base=1000 * rank)

    peak, peak_kind = measured_peak_gbs()
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 query/sink/tail; u4 keys and u2 values dequantised to fp16 operands, fp32 accumulate",
        "data": "synthetic",
        "config": {"workload": "config 1: Qwen2.5-7B-shaped single-request decode, 28 layers x 4 KV heads x 128, 28 query heads, "
                               "32768-token history packed K4/V2 (127 blocks of 256), bf16 sink 4 + tail 252 growing by 1/step",
                   "requests_per_gpu": 1, "launch": "CUDA graph of one launch (decode with the append of the new token fused in)" if use_graph else "eager, one launch per step", "l2": "inputs larger than L2 (402 MB read per step vs 126 MB L2)",
                   "sharding": "one request per GPU, no collective" if world > 1 else "single GPU"},
        "us_per_step": round(ms_per_step * 1e3, 2),
        "packed_gbs": round(world * (mean_bytes["packed"] + mean_bytes["metadata"]) / (ms_per_step * 1e-3) / 1e9, 1),
        "algorithmic_bytes_per_step": {k: int(v) for k, v in mean_bytes.items()},
        "encode_tokens_per_s": round(world * CONTEXT / (encode_ms * 1e-3), 1),
        "encode_ms_all_layers": round(encode_ms, 3),
        "append": append_info,
        "encode_kernels": {"us_per_layer": round(encode_kernels_us, 1),
                           "tokens_per_s_all_layers": round(world * CONTEXT / (encode_kernels_us * 1e-6 * LAYERS), 1),
                           "hbm_frac": round((blocks_bytes_encode() / (encode_kernels_us * 1e-6) / 1e9) / measured_peak_gbs()[0], 4),
                           "what": "K4 + V2 encoder launches of one layer back to back through the C ABI, device time"},
        "roofline": {"bound": "hbm", "kernel": "decode_kernel", "achieved": round(achieved, 1), "peak": peak,
                     "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_source": peak_kind,
                     "us_per_launch": round(kernel_ms * 1e3, 2),
                     "traffic": int(kernel_bytes * DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE) if DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE else None,
                     "traffic_source": DECODE_TRAFFIC_SOURCE},
        "e2e": {"value": round(world * mean_bytes["total"] / (e2e_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
                "us_per_step": round(e2e_ms * 1e3, 2), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,   # decode launches of this library, one per step (torch's staging copy not counted)
        "clocks": clocks.summary(),
        "device_status": status,
        "parity": parity,
    }
    if sustained is not None:
        peak_now = measured_peak_gbs()[0]
        sustained["gbs"] = round(kernel_bytes / (sustained["us_per_step"] * 1e-6) / 1e9, 1)
        sustained["frac"] = round(sustained["gbs"] / peak_now, 4)
        burst_mhz = line["clocks"]["sm_mhz"] or line["clocks"]["sm_max_mhz"]
        sustained["burst_us_times_mhz"] = round(ms_per_step * 1e3 * burst_mhz, 0) if burst_mhz else None
        line["sustained"] = sustained
    if not args.no_append_sequence:
        # DecodeBatch advanced the tails on the device only: the cache's own counters still describe the prefill
        line["append_sequence"] = append_sequence_leg(torch, device, cache)
    if args.split_context:
        del batch, cache
        torch.cuda.empty_cache()
        line["split_kv"] = run_split_kv(args, torch, dist, device, world, rank)
    if world == 1 and not args.no_prefill:
        line["prefill"] = run_prefill(torch, device)
    if not args.no_paged_batch:
        torch.cuda.empty_cache()
        line["paged_batch"] = run_paged_batch(torch, dist, device, world, rank, 16)
        torch.cuda.empty_cache()
        # the same requests with the reference's 64-token pages, for comparison
        line["paged_batch"]["pages_of_64_tokens"] = {
            k: v for k, v in run_paged_batch(torch, dist, device, world, rank, 64).items()
            if k in ("us_per_step", "decode_tokens_per_s", "aggregate_gbs", "per_gpu_hbm_frac", "algorithmic_bytes_per_step", "parity")}
    if world == 1 and args.model_step:
        torch.cuda.empty_cache()
        line["model_step"] = run_model_step(args, torch, device)
    if rank == 0 and world == 1 and not args.no_value_codecs:
        torch.cuda.empty_cache()
        line["value_codecs"] = value_codecs_leg(torch, device)
    if rank == 0 and world == 1 and not args.no_reference_gpu:
        torch.cuda.empty_cache()
        try:
            line["reference_gpu"] = reference_gpu_leg(torch, device)
        except Exception as exc:   # the reference's kernels are JIT-compiled on the spot: report, do not fail the run
            line["reference_gpu"] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(sample_layers=1)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_model_step(args, torch, device):
    """Opt-in leg: one decode token of a randomly initialised Qwen2.5-7B-shaped model (28 layers,
    hidden 3584, 28/4 heads of 128, vocabulary 152064, bf16) over a 32768-token packed cache,
    through the model adapter layer by layer (eager) and as one replayed CUDA graph."""
    import time
    import workloads
    from transformers import Qwen2Config, Qwen2ForCausalLM
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.graph_decode import GraphedDecodeStep
    from inquant.qwen_fused import enable_fused_attention
    config = Qwen2Config(vocab_size=152064, hidden_size=Q_HEADS * DIM, intermediate_size=18944, head_dim=DIM,
                         num_hidden_layers=LAYERS, num_attention_heads=Q_HEADS, num_key_value_heads=KV_HEADS,
                         max_position_embeddings=131072, attn_implementation="sdpa")
    previous = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            model = Qwen2ForCausalLM(config).eval()
    finally:
        torch.set_default_dtype(previous)
    weight_bytes = sum(p.numel() * p.element_size() for p in model.parameters())
    context = CONTEXT
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=BLOCK, residual_length=RESIDUAL,
                                     sink_tokens=SINK, value_bits=2, value_group_size=64, validate_positions=False))
    for layer in range(LAYERS):   # the history is synthetic: the adapter only needs a filled cache
        k, v = workloads.make_kv_torch(70000 + layer, KV_HEADS, context, device)
        cache.update(k, v, layer)
        del k, v
    result = {"workload": f"config 1 shapes with the model around the attention: {LAYERS}-layer Qwen2.5-7B-shaped random-init "
                          f"model, {context}-token packed history, batch 1, greedy decode",
              "weights_gb": round(weight_bytes / 1e9, 2)}
    with enable_fused_attention(model), torch.no_grad():
        token = torch.tensor([[17]], device=device)
        for _ in range(3):
            model(token, past_key_values=cache)
        torch.cuda.synchronize()
        steps = 20
        t0 = time.perf_counter()
        for _ in range(steps):
            model(token, past_key_values=cache)
        torch.cuda.synchronize()
        result["eager_ms_per_token"] = round((time.perf_counter() - t0) / steps * 1e3, 3)
        stepper = GraphedDecodeStep(model, cache)
        stepper.step(17)
        for _ in range(3):
            stepper.step()
        torch.cuda.synchronize()
        steps = 60
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            stepper.step()
        e1.record()
        torch.cuda.synchronize()
        result["graphed_ms_per_token"] = round((time.perf_counter() - t0) / steps * 1e3, 3)
        result["graphed_device_ms_per_token"] = round(e0.elapsed_time(e1) / steps, 3)
        result["graph_replays"], result["eager_seal_steps"] = stepper.replays, stepper.eager_steps
        stepper.close()
    peak, _ = measured_peak_gbs()
    kv_bytes = LAYERS * KV_HEADS * ((CONTEXT - SINK - RESIDUAL) // BLOCK) * BLOCK * 104
    result["hbm_floor_ms"] = round((weight_bytes + kv_bytes) / (peak * 1e9) * 1e3, 3)
    result["hbm_frac_graphed"] = round(result["hbm_floor_ms"] / result["graphed_device_ms_per_token"], 4)
    del model, cache
    torch.cuda.empty_cache()
    return result


def run_prefill(torch, device):
    """Config 2, one of the 28 layers: the 32768-token prompt arrives as 16 chunks of 2048; every
    chunk attends to the cache's history (dequantised by this library's kernels into dense
    tensors) plus itself with the tcgen05 kernel, then is sealed into the packed cache.  Reports
    the whole chunk loop through the public API and the attention kernel alone."""
    import workloads
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.prefill import PrefillHistory, prefill_attention, prefill_chunk
    chunk = 2048
    k, v = workloads.make_kv_torch(4242, KV_HEADS, CONTEXT, device)
    gen = torch.Generator(device=device).manual_seed(99)
    q = torch.randn((1, Q_HEADS, CONTEXT, DIM), device=device, generator=gen).bfloat16()
    cfg = CacheConfig(CodecConfig(donor_policy="min_error", donor_backend="triton"), block_size=BLOCK,
                      residual_length=RESIDUAL, sink_tokens=SINK, value_bits=2, value_group_size=64, validate_positions=False)
    scale = DIM ** -0.5
    flops = sum(4 * Q_HEADS * DIM * (chunk * c0 + chunk * (chunk + 1) // 2) for c0 in range(0, CONTEXT, chunk))

    def whole_layer(persistent=False):
        cache = InQuantCache(cfg)
        history = PrefillHistory(cache, CONTEXT, persistent=persistent)
        for c0 in range(0, CONTEXT, chunk):
            prefill_chunk(cache, q[:, :, c0:c0 + chunk], k[:, :, c0:c0 + chunk], v[:, :, c0:c0 + chunk], 0, scale,
                          history=history)
        history.check()
    for _ in range(2):
        whole_layer()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        whole_layer()
    e1.record()
    torch.cuda.synchronize()
    layer_ms = e0.elapsed_time(e1) / 3
    whole_layer(True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(3):
        whole_layer(True)
    e1.record()
    torch.cuda.synchronize()
    layer_ms_persistent = e0.elapsed_time(e1) / 3
    # the attention kernel alone on the last (largest) chunk: 2048 queries over 32768 keys
    out = torch.empty((1, Q_HEADS, chunk, DIM), dtype=torch.bfloat16, device=device)
    last_q = q[:, :, CONTEXT - chunk:]
    for _ in range(3):
        prefill_attention(last_q, k, v, scale, out=out)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(10):
        prefill_attention(last_q, k, v, scale, out=out)
    e1.record()
    torch.cuda.synchronize()
    kernel_ms = e0.elapsed_time(e1) / 10
    kernel_flops = 4 * Q_HEADS * DIM * (chunk * (CONTEXT - chunk) + chunk * (chunk + 1) // 2)
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
        burst, sustained, source = float(peaks["bf16_tflops"]), float(peaks["bf16_tflops_sustained"]), "measured"
    except Exception:
        burst, sustained, source = 1590.0, 1400.0, "fallback"
    kernel_tflops = kernel_flops / (kernel_ms * 1e-3) / 1e12
    return {
        "workload": "config 2, one layer: 16 chunks of 2048 tokens over the packed history (K4/V2), 28 query heads, bf16",
        "layer_ms": round(layer_ms, 3), "layer_tflops": round(flops / (layer_ms * 1e-3) / 1e12, 1),
        "layer_includes": "per chunk: the layer's history rebuilt from the packed cache into one scratch pair shared by all layers (71 MB "
                          "for a 32768-token prompt; no dense copy is kept), the attention kernel, sealing the chunk",
        "layer_ms_with_persistent_dense_history": round(layer_ms_persistent, 3),
        "tokens_per_s_all_layers": round(CONTEXT / (layer_ms * 1e-3 * LAYERS), 1),
        "roofline": {"bound": "tensor", "kernel": "prefill_kernel (2048 queries over 32768 keys)", "achieved": round(kernel_tflops, 1),
                     "peak": burst, "unit": "TFLOP/s", "frac": round(kernel_tflops / burst, 4),
                     "frac_of_sustained": round(kernel_tflops / sustained, 4), "peak_source": source,
                     "us_per_launch": round(kernel_ms * 1e3, 1)},
    }


def run_paged_batch(torch, dist, device, world, rank, block):
    """Config 3: Mistral-7B-shaped batched paged decode (vLLM-extension page layout, block 16):
    32 layers x 8 KV heads x 128, 32 query heads, 16 requests with seeded context lengths uniform
    in 4096..32768, pages at shuffled physical ids, requests dealt to the ranks by context length with no
    collective.  One step = every layer of every local request in one decode launch.  A request's
    pages are sealed once by the page-packing kernels and copied to the other layers' (distinct)
    physical pages, so every layer still streams its own memory."""
    import numpy as np
    import workloads
    from inquant.batched import DecodeBatch, PagedSequenceState, shard_requests
    from inquant_vllm.layout import PageLayout, pack_pages_into
    layers, heads, q_heads, requests = 32, 8, 32, 16
    layout = PageLayout(block, heads)
    lengths = [int(x) for x in np.random.default_rng(2024).integers(4096, 32769, size=requests)]
    mine = shard_requests(lengths, world)[rank]
    pages_of = {i: lengths[i] // block for i in mine}
    total_pages = layers * sum(pages_of.values())
    pool = torch.empty((total_pages + 8, layout.page_bytes), dtype=torch.uint8, device=device)
    order = torch.randperm(total_pages + 8, generator=torch.Generator().manual_seed(7 + rank)).to(device=device, dtype=torch.int32)
    cursor, seqs = 0, []
    for i in mine:
        n, pages = lengths[i], pages_of[i]
        k, v = workloads.make_kv_torch(9000 + i, heads, n, device)
        tail, sink = n % block, min(4, n)
        dense = torch.zeros((2, heads, block + 4, DIM), dtype=torch.bfloat16, device=device)
        dense[0, :, :sink], dense[1, :, :sink] = k[0, :, :sink], v[0, :, :sink]
        if tail:
            dense[0, :, 4:4 + tail], dense[1, :, 4:4 + tail] = k[0, :, n - tail:], v[0, :, n - tail:]
        kt = k[0, :, :pages * block].reshape(heads, pages, block, DIM).permute(1, 0, 2, 3).contiguous()
        vt = v[0, :, :pages * block].reshape(heads, pages, block, DIM).permute(1, 0, 2, 3).contiguous()
        first = order[cursor:cursor + pages].contiguous()
        pack_pages_into(kt, vt, layout, pool, first)
        for layer in range(layers):
            ids = order[cursor:cursor + pages].contiguous()
            cursor += pages
            if layer:
                pool[ids.long()] = pool[first.long()]
            seqs.append(PagedSequenceState(pool, ids, pages, dense.clone(), tail, sink, layout))
        del k, v, kt, vt
    batch = DecodeBatch(seqs, q_heads, torch.bfloat16)
    gen = torch.Generator(device=device).manual_seed(31 + rank)
    batch.queries.copy_(torch.randn(batch.queries.shape, device=device, generator=gen).to(torch.bfloat16))
    for _ in range(3):
        batch.attend()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    steps = 20
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        batch._launch_attend()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    parity = check_paged_parity(torch, batch, seqs, [lengths[i] for i in mine], layers, block, heads)
    total_bytes = batch.algorithmic_bytes()["total"]
    if world > 1:
        t = torch.tensor([ms, float(total_bytes)], device=device, dtype=torch.float64)
        worst = t.clone()
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, total_bytes = float(worst[0].item()), float(t[1].item())
    peak, _ = measured_peak_gbs()
    gbs = total_bytes / (ms * 1e-3) / 1e9
    return {"workload": f"config 3: 16 requests x 32 layers, 8 KV heads, 32 query heads, contexts 4096..32768, pages of {block} tokens",
            "requests": requests, "context_tokens": sum(lengths), "us_per_step": round(ms * 1e3, 1),
            "decode_tokens_per_s": round(requests / (ms * 1e-3), 1), "aggregate_gbs": round(gbs, 1),
            "per_gpu_hbm_frac": round(gbs / world / peak, 4), "algorithmic_bytes_per_step": int(total_bytes),
            "sharding": "requests dealt to the ranks by context length (longest first, to the least loaded rank), no collective", "steps": steps,
            "parity": parity}


def run_split_kv(args, torch, dist, device, world, rank):
    """Config 4: one 131072-token request, sealed blocks partitioned by sequence over the ranks,
    partial (acc, m, l) records exchanged once per step (peer-memory kernel when the ranks can
    map one another's inbox, else an all-gather) and merged."""
    import workloads
    from inquant.cache import CacheConfig, InQuantCache
    from inquant.codec import CodecConfig
    from inquant.batched import SequenceState
    from inquant import _native as N
    from inquant.split_kv import SplitKVDecode, shard_blocks
    context = args.split_context
    total_blocks = (context - SINK - RESIDUAL) // BLOCK
    start, end = shard_blocks(total_blocks, world, rank)
    first, last = rank == 0, rank == world - 1
    tail = context - SINK - total_blocks * BLOCK
    tokens = (SINK if first else 0) + (end - start) * BLOCK + (tail if last else 0)
    cache = InQuantCache(CacheConfig(CodecConfig(donor_policy="min_error"), block_size=BLOCK,
                                     residual_length=RESIDUAL if last else 0, sink_tokens=SINK if first else 0,
                                     value_bits=2, value_group_size=64, validate_positions=False))
    for layer in range(LAYERS):
        k, v = workloads.make_kv_torch(50000 + 1000 * rank + layer, KV_HEADS, tokens, device)
        cache.update(k, v, layer)
        del k, v
    seqs = [SequenceState.from_cache_layer(cache, i) for i in range(LAYERS)]
    assert all(len(s.decode_state.key_blocks) == end - start for s in seqs)
    gen = torch.Generator(device=device).manual_seed(99)   # the same queries on every rank
    steps = min(args.steps, 40)
    inputs = torch.randn((args.warmup + steps, LAYERS, Q_HEADS + 2 * KV_HEADS, DIM), device=device, generator=gen).bfloat16()
    use_graph = not args.no_graph

    parity = {}

    def time_split(exchange, check=False):
        split = SplitKVDecode(seqs, Q_HEADS, owns_tail=last, exchange=exchange)
        for i in range(args.warmup):
            split.inputs.copy_(inputs[i])
            split.step()
        torch.cuda.synchronize()
        if use_graph:
            split.capture()
            split.inputs.copy_(inputs[0])
            split.replay()
        run_step = split.replay if use_graph else split.step
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(steps):
            split.inputs.copy_(inputs[args.warmup + i])
            run_step()
        t1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / steps
        if check:
            parity[exchange] = check_split_parity(torch, dist, split, cache, run_step, inputs[0], world, rank, first, last)
        local_bytes = split.batch.algorithmic_bytes()["total"]
        stats = torch.tensor([ms, float(local_bytes)], device=device, dtype=torch.float64)
        if world > 1:
            worst = stats.clone()
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            total = stats.clone()
            dist.all_reduce(total, op=dist.ReduceOp.SUM)
            return float(worst[0]), float(total[1]), split.exchange
        return ms, float(local_bytes), split.exchange

    record_bytes = LAYERS * Q_HEADS * 130 * 4
    describe = {
        "fused": (f"inside the decode launch: the CTA that merges a (layer, KV head) pair stores its records ({record_bytes} B per rank "
                  "and step in all) into every peer's inbox over NVLink peer memory, every word as one 8-byte store tagged with the "
                  "step number (no fence, no flags), polls the peers' words (bounded) and merges all ranks' records",
                  "CUDA graph of ONE launch per rank (decode with the append fused in on the tail owner and the exchange in its merge)"),
        "p2p": (f"peer memory: one kernel per rank stores its {record_bytes} B of records into every peer's inbox over "
                "NVLink, signals, waits (bounded) and merges",
                "CUDA graph of decode (append fused in on the tail owner) + one exchange-and-merge kernel"),
        "nccl": (f"one all-gather of {record_bytes} B per rank per step, then a local log-sum-exp merge",
                 "CUDA graph of decode (append fused in on the tail owner) + all-gather + merge"),
    }
    # every exchange this node offers is timed (each with its own parity check); the fastest is the
    # leg's figure and the others are reported beside it
    timed = {}
    for name in args.split_exchanges.split(","):
        if name == "nccl" or world == 1:
            if "nccl" not in timed:
                timed["nccl"] = time_split("nccl", check=True)
            continue
        try:
            result = time_split(name, check=name not in parity)
        except RuntimeError:
            continue   # every rank raises alike: the peer mappings are agreed on collectively
        # an exchange named twice is timed twice (the order of the legs is then visible in the figures)
        timed[name if name not in timed else name + "_again"] = result
    best = min(timed, key=lambda name: timed[name][0])
    ms, total_bytes, exchange = timed[best]
    how, launch = describe[best.replace("_again", "")]
    if not use_graph:
        launch = "eager"
    extra = {"us_per_step_by_exchange": {name: round(t[0] * 1e3, 2) for name, t in timed.items()}}
    if N.take_status(device):
        raise RuntimeError("a split-KV kernel reported a failure in the status word")
    peak, _ = measured_peak_gbs()
    return {"context": context, "blocks_per_rank": end - start, "us_per_step": round(ms * 1e3, 2),
            "aggregate_gbs": round(total_bytes / (ms * 1e-3) / 1e9, 1),
            "per_gpu_hbm_frac": round(total_bytes / world / (ms * 1e-3) / 1e9 / peak, 4),
            "exchange": how, "launch": launch,
            "steps": steps, "parity": dict(parity[best.replace("_again", "")], exchanges_checked=sorted(parity)), **extra}


# DRAM bytes (read + write) of one decode_kernel launch per algorithmic byte, from one ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum) of a 10-layer case of the same kernel, scaled to the
# layers of this run because traffic grows in proportion to the units processed.  The source string
# names the capture; set the ratio to None when the kernel changes and no new capture exists.
DECODE_TRAFFIC_PER_ALGORITHMIC_BYTE = 150.17 / 143.72
DECODE_TRAFFIC_SOURCE = ("ncu capture of the 10-layer case (145.49 MB read + 4.68 MB written against 143.72 MB algorithmic) of "
                         "the decode kernel as it stands (whole-slice fast path, fragment-product fold, fused append), scaled by units")


# --------------------------------------------------------------------------- CPU arm (oracle port)
def cpu_layer(seed):
    """Encode one layer of the workload with the CPU oracle; returns what its decode needs."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import inquant_oracle as oracle
    import workloads
    k, v = workloads.make_kv(seed, KV_HEADS, CONTEXT, outliers=6, adjacent=3)
    take, blocks, tail = oracle.seal_plan(0, 0, CONTEXT, sink_tokens=SINK, residual_length=RESIDUAL, block_size=BLOCK)
    body = slice(take, take + blocks * BLOCK)
    shape = (KV_HEADS, blocks, BLOCK, DIM)
    kb = np.ascontiguousarray(k[0][:, body].reshape(shape).transpose(1, 0, 2, 3))
    vb = np.ascontiguousarray(v[0][:, body].reshape(shape).transpose(1, 0, 2, 3))
    t0 = time.perf_counter()
    pk = oracle.quantize_k4(kb, "bfloat16", 8, 0.125, "min_error")
    pv = oracle.quantize_values(vb, "bfloat16", 2, 64)
    encode_s = time.perf_counter() - t0
    dense = (k[0][:, :take], v[0][:, :take], k[0][:, take + blocks * BLOCK:], v[0][:, take + blocks * BLOCK:])
    return oracle, pk, pv, dense, blocks, encode_s


def cpu_decode_once(oracle, pk, pv, dense, q):
    import numpy as np
    sk, sv, tk, tv = dense
    keys = oracle.dequantize_k4(pk).transpose(1, 0, 2, 3).reshape(KV_HEADS, -1, DIM)
    vals = oracle.dequantize_values(pv).transpose(1, 0, 2, 3).reshape(KV_HEADS, -1, DIM)
    keys = np.concatenate([sk, keys, tk], 1)
    vals = np.concatenate([sv, vals, tv], 1)
    return oracle.attention_decode(q, keys, vals, DIM ** -0.5)


_POOL_STATE = {}


def _cpu_partition(task):
    """One partition of the layer on one host core: dequantise blocks [b0, b1) (plus the exact sink
    on the first partition and the exact tail on the last) and return the partial record."""
    import numpy as np
    b0, b1, first, last = task
    if not _POOL_STATE.get("limited"):
        try:   # one BLAS thread per worker: the workers are the parallelism
            from threadpoolctl import threadpool_limits
            _POOL_STATE["limiter"] = threadpool_limits(1)
        except Exception:
            pass
        _POOL_STATE["limited"] = True
    oracle, pk, pv, dense, q = (_POOL_STATE[k] for k in ("oracle", "pk", "pv", "dense", "q"))
    sk, sv, tk, tv = dense
    part_k = oracle.PackedK(**{n: a[b0:b1] for n, a in pk.fields().items()}, shape=(b1 - b0, *pk.shape[1:]), dtype=pk.dtype)
    part_v = oracle.PackedV(**{n: a[b0:b1] for n, a in pv.fields().items()}, shape=(b1 - b0, *pv.shape[1:]), dtype=pv.dtype,
                            bits=pv.bits, group_size=pv.group_size)
    keys = oracle.dequantize_k4(part_k).transpose(1, 0, 2, 3).reshape(KV_HEADS, -1, DIM)
    vals = oracle.dequantize_values(part_v).transpose(1, 0, 2, 3).reshape(KV_HEADS, -1, DIM)
    if first:
        keys, vals = np.concatenate([sk, keys], 1), np.concatenate([sv, vals], 1)
    if last:
        keys, vals = np.concatenate([keys, tk], 1), np.concatenate([vals, tv], 1)
    return oracle.attention_partial(q, keys, vals, DIM ** -0.5)


class CpuDecoder:
    """The CPU arm on every host core: the layer's blocks are cut into one partition per core
    (forked workers share the packed arrays), partial records are merged as the reference's
    split kernel merges them."""

    def __init__(self, oracle, pk, pv, dense, q, blocks):
        import multiprocessing
        self.cores = max(1, min(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count(), blocks))
        _POOL_STATE.update(oracle=oracle, pk=pk, pv=pv, dense=dense, q=q)
        self.oracle = oracle
        edges = [blocks * i // self.cores for i in range(self.cores + 1)]
        self.tasks = [(edges[i], edges[i + 1], i == 0, i == self.cores - 1) for i in range(self.cores)]
        self.pool = multiprocessing.get_context("fork").Pool(self.cores) if self.cores > 1 else None

    def step(self):
        import numpy as np
        parts = self.pool.map(_cpu_partition, self.tasks) if self.pool else [_cpu_partition(t) for t in self.tasks]
        acc, m, l = (np.stack([p[i] for p in parts]) for i in range(3))
        return self.oracle.merge_partials(acc, m, l)

    def close(self):
        if self.pool:
            self.pool.close()
            self.pool.join()


def layer_bytes(blocks, tail):
    return (KV_HEADS * blocks * BLOCK * 104 + KV_HEADS * blocks * 608 + (SINK + tail) * KV_HEADS * DIM * 2 * 2
            + Q_HEADS * DIM * 2 * 2)


def cpu_baseline(sample_layers=1, repeats=3):
    """The CPU arm, run in a process of its own (it forks one worker per host core, which a
    process that holds a CUDA context should not do) and reported as this line's cpu_baseline."""
    import subprocess
    env = dict(os.environ)
    for name in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(name, None)
    done = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference", "--steps", str(repeats),
                           "--warmup", "1"], capture_output=True, text=True, env=env, timeout=900)
    line = json.loads(done.stdout.strip().splitlines()[-1])
    base = line["cpu_baseline"]
    base["us_per_step_extrapolated"] = round(line["ms_per_step"] * LAYERS * 1e3, 1)
    base["encode_tokens_per_s"] = line["encode_tokens_per_s"]
    return base


def _reference_modules():
    """The unmodified reference packages installed under oracle/_ref by oracle/build_ref.py, imported
    under another name (this repository's mirror is also called `inquant`); None when absent."""
    import importlib
    path = os.path.join(ROOT, "oracle")
    if path not in sys.path:
        sys.path.insert(0, path)
    try:
        import build_ref
        if not build_ref.available():
            return None
        build_ref.load_reference()
        names = ("codec", "value_codec", "cache", "qwen_fused")
        return {name: importlib.import_module(f"inquant_reference.{name}") for name in names}
    except Exception:
        return None


def run_reference_torch(args, ref, world):
    """The reference's own torch CPU implementation of the path, unmodified, on all host cores:
    `InQuantCache.update` seals one layer of config 1 (32768 tokens, 4 KV heads); a step is that
    layer's decode as the reference's oracle does it -- `append_for_attention`, then
    `_reference_decode` (dequantise every block, SDPA with grouped queries)."""
    import torch
    import workloads
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    codec, cache_mod, fused = ref["codec"], ref["cache"], ref["qwen_fused"]
    k32, v32 = workloads.make_kv(0, KV_HEADS, CONTEXT, outliers=6, adjacent=3)
    k, v = torch.from_numpy(k32).to(torch.bfloat16), torch.from_numpy(v32).to(torch.bfloat16)
    config = cache_mod.CacheConfig(codec.CodecConfig(donor_policy="min_error"), block_size=BLOCK, residual_length=RESIDUAL,
                                   sink_tokens=SINK, value_bits=2, value_group_size=64, validate_positions=False)
    cache = cache_mod.InQuantCache(config)
    t0 = time.perf_counter()
    cache.update(k, v, 0)
    encode_s = time.perf_counter() - t0
    gen = torch.Generator().manual_seed(3)
    q = torch.from_numpy(workloads.make_query(0, Q_HEADS)).to(torch.bfloat16).view(1, Q_HEADS, 1, DIM)
    scale = DIM ** -0.5

    def step():
        new_k = torch.randn((1, KV_HEADS, 1, DIM), generator=gen).to(torch.bfloat16)
        new_v = torch.randn((1, KV_HEADS, 1, DIM), generator=gen).to(torch.bfloat16)
        view = cache.append_for_attention(new_k, new_v, 0)
        return fused._reference_decode(q, view, scale), view

    t0 = time.perf_counter()
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    once = (time.perf_counter() - t0) / max(1, min(args.warmup, 2))
    # a bounded sample: about a minute of host time, and no block seal inside the timed steps
    steps = max(1, min(args.steps, int(60.0 / max(once, 1e-3)), 100))
    t0 = time.perf_counter()
    for _ in range(steps):
        _, view = step()
    per = (time.perf_counter() - t0) / steps
    blocks, tail = len(view.key_blocks), view.residual_key.shape[2]
    nbytes = layer_bytes(blocks, tail)
    value = round(nbytes / per / 1e9, 4)
    sample = (f"each step = ONE of the 28 layers (32768 tokens, 4 KV heads) through the reference's own torch CPU path "
              f"(append_for_attention + _reference_decode: dequantise {blocks} blocks, SDPA), {cores} torch threads, "
              f"{steps} timed steps of {per * 1e3:.0f} ms; GB/s is per byte, so not scaled")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": max(1, min(args.warmup, 2)), "ms_per_step": round(per * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 dequantised K/V, torch CPU SDPA", "data": "synthetic",
        "config": {"workload": "config 1 (one layer per step on the host cores)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "reference", "sample": sample,
                         "torch_threads": torch.get_num_threads(), "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "encode_tokens_per_s": round(CONTEXT / (encode_s * LAYERS), 1),
        "encode_ms_one_layer": round(encode_s * 1e3, 1),
    }))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    ref = None if args.reference_port else _reference_modules()
    if ref is not None:
        return run_reference_torch(args, ref, world)
    import workloads
    oracle, pk, pv, dense, blocks, encode_s = cpu_layer(0)
    q = workloads.make_query(0, Q_HEADS)
    decoder = CpuDecoder(oracle, pk, pv, dense, q, blocks)
    # one warm-up step each way; the timed steps use whichever is faster on this host (one process
    # whose BLAS may use all cores, or one partition per core)
    t0 = time.perf_counter()
    cpu_decode_once(oracle, pk, pv, dense, q)
    single = time.perf_counter() - t0
    decoder.step()
    t0 = time.perf_counter()
    decoder.step()
    partitioned = time.perf_counter() - t0
    use_pool = partitioned < single
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(steps):
        decoder.step() if use_pool else cpu_decode_once(oracle, pk, pv, dense, q)
    per = (time.perf_counter() - t0) / steps
    decoder.close()
    cores = decoder.cores if use_pool else 1
    nbytes = layer_bytes(blocks, dense[2].shape[1])
    value = round(nbytes / per / 1e9, 4)
    sample = ("each step = ONE of the 28 layers (32768 tokens, 4 KV heads): numpy restatement of the reference's torch CPU "
              f"path (dequantise all blocks + attention), "
              + (f"cut into one partition per host core ({decoder.cores} workers)" if use_pool else
                 f"in one process (faster here than {decoder.cores} partition workers: {single:.2f} s vs {partitioned:.2f} s)")
              + f", {steps} timed steps; GB/s is per byte, so not scaled")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": min(args.warmup, 1), "ms_per_step": round(per * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64 attention over bf16-rounded dequantised K/V", "data": "synthetic",
        "config": {"workload": "config 1 (one layer per step on the host cores)"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "encode_tokens_per_s": round(CONTEXT / (encode_s * LAYERS), 1),
    }))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=128)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="cuda", choices=("cuda", "reference"))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-graph", action="store_true", help="launch the two kernels eagerly instead of replaying a CUDA graph")
    parser.add_argument("--split-context", type=int, default=131072,
                        help="also time config 4: one request of this many tokens split by sequence over the ranks (0 = skip)")
    parser.add_argument("--layers", type=int, default=LAYERS, help="fewer layers for profiler captures (default: the full 28)")
    parser.add_argument("--skip-e2e", action="store_true", help="profiler captures: skip the host-buffer leg")
    parser.add_argument("--no-prefill", action="store_true", help="skip the chunked-prefill leg (config 2, one layer)")
    parser.add_argument("--no-paged-batch", action="store_true", help="skip the batched paged decode leg (config 3)")
    parser.add_argument("--reference-port", action="store_true",
                        help="--impl reference: time the numpy port of the reference even when oracle/_ref holds the reference itself")
    parser.add_argument("--no-append-sequence", action="store_true",
                        help="skip the 136-step append sequence that crosses a block seal (config 1)")
    parser.add_argument("--split-exchanges", default="fused,p2p,nccl",
                        help="exchanges of the split-KV leg to time, in this order (fused, p2p, nccl; several GPUs only)")
    parser.add_argument("--no-value-codecs", action="store_true", help="skip the one-layer leg over the other value codecs")
    parser.add_argument("--no-reference-gpu", action="store_true",
                        help="skip the leg that runs the reference's Triton decode kernel beside this library's")
    parser.add_argument("--sustained-seconds", type=float, default=2.5,
                        help="length of the sustained-clock leg (0 = skip)")
    parser.add_argument("--model-step", action="store_true",
                        help="also time a whole-model decode token (random-init 7B-shaped model) eagerly and from one CUDA graph")
    args = parser.parse_args()
    globals()["LAYERS"] = args.layers
    args.warmup = max(args.warmup, 3) if args.impl == "cuda" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
