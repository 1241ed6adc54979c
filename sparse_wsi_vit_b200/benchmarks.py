"""Secondary workloads of the sparse-attention path, timed on one GPU with CUDA events.

    python bench.py --workload block_sparse     # 2-D block-sparse sweep: H=16, D=128, block 128
    python bench.py --workload nsa              # NSA-style attention, 65536 tokens, 16 q / 2 kv heads, D=128
    python bench.py --workload encoder          # 12-layer DSA slide encoder (d=768, 12x64, top-2048) on 4 slide sizes
    python bench.py --workload static           # 2-layer static-pattern encoder (d=384, 6x64), 4096 tokens

Each prints one JSON line per configuration.  The default workload of bench.py (the DSA forward at
65536 tokens) is the headline number; these lines are the other configurations of the same path.
Inputs are seeded synthetic tensors of the stated shapes; weights are seeded random initialisations.
"""
from __future__ import annotations

import json
import os
import statistics

import numpy as np
import torch


def _peak_tflops():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("bf16_tflops_sustained", 1411.6), "measured"
    return 1400.0, "fallback"


def _time_ms(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return statistics.median(a.elapsed_time(b) for a, b in ev)


def block_sparse_sweep(steps=5, warmup=3, max_pflop=8.0, sizes=(8192, 32768, 131072, 262144), ps=(0.01, 0.05, 0.25)):
    """Band +-2 blocks, one global block, Bernoulli(p) extra key blocks per query block."""
    from . import ops
    from .patterns import band_random_blocks
    dev = torch.device("cuda", 0)
    H, D, BS = 16, 128, 128
    peak, src = _peak_tflops()
    g = torch.Generator().manual_seed(0)
    for n in sizes:
        q, k, v = (torch.randn(1, H, n, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
        for p in ps:
            rp, ci = band_random_blocks(n // BS, band=2, n_global=1, p=p, seed=1)
            nnz = int(rp[-1])
            flops = 4.0 * BS * BS * nnz * H * D
            line = {"workload": "block_sparse", "tokens": n, "heads": H, "head_dim": D, "block": BS, "p_extra": p,
                    "nnz_blocks": nnz, "density": nnz / float((n // BS) ** 2), "flops": flops}
            if flops > max_pflop * 1e15:
                line["skipped"] = f"more than {max_pflop} PFLOP per step"
                print(json.dumps(line), flush=True)
                continue
            rpd, cid = torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev)
            ms = _time_ms(lambda: ops.block_sparse_attention(q, k, v, rpd, cid, BS), steps, warmup)
            ops.check_status(dev, "block_sparse sweep")
            tf = flops / (ms * 1e-3) / 1e12
            line.update({"ms": ms, "tokens_per_s": n / (ms * 1e-3), "tflops": tf, "frac_of_bf16_peak": tf / peak,
                         "peak_source": f"bf16_tflops_sustained of {src}", "dense_flops": 4.0 * n * n * H * D})
            print(json.dumps(line), flush=True)
        del q, k, v


def nsa_forward(steps=3, warmup=1, tokens=65536):
    from . import ops
    from .nsa import nsa_attention
    dev = torch.device("cuda", 0)
    Hq, Hkv, D = 16, 2, 128
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, Hq, tokens, D, generator=g).to(torch.bfloat16).to(dev)
    k = torch.randn(1, Hkv, tokens, D, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(1, Hkv, tokens, D, generator=g).to(torch.bfloat16).to(dev)
    gate = torch.randn(1, tokens, Hq, 3, generator=g).to(dev)
    ms = _time_ms(lambda: nsa_attention(q, k, v, gate), steps, warmup)
    ops.check_status(dev, "nsa forward")
    n_c = (tokens - 32) // 16 + 1
    flops = 4.0 * tokens * Hq * D * (n_c + 16 * 64 + 513)
    print(json.dumps({"workload": "nsa_fwd", "tokens": tokens, "q_heads": Hq, "kv_heads": Hkv, "head_dim": D,
                      "compress": "mean 32/16", "select": "16 blocks of 64", "window": 512, "ms": ms,
                      "tokens_per_s": tokens / (ms * 1e-3), "branch_flops": flops,
                      "tflops": flops / (ms * 1e-3) / 1e12}), flush=True)


def encoder_slides(steps=2, warmup=1, sizes=(24576, 57344, 98304, 131072)):
    """12 x (DSA block d=768, 12 heads x 64, MLP 3072, top-2048, 4 x 64 indexer), bf16 autocast."""
    from . import DSAViTSlideEncoder, ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    net = DSAViTSlideEncoder(in_features=1280, out_features=2, embed_dim=768, num_heads=12, num_layers=12, num_cls=2,
                             indexer_heads=4, indexer_dim=64, top_k=2048).to(dev).eval()
    g = torch.Generator().manual_seed(1)
    for n in sizes:
        x = torch.randn(1, n, 1280, generator=g).to(torch.bfloat16).to(dev)

        def fwd():
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                return net(x)["logits"]

        ms = _time_ms(fwd, steps, warmup)
        ops.check_status(dev, "encoder forward")
        print(json.dumps({"workload": "dsa_encoder_12l", "tokens": n, "embed_dim": 768, "heads": 12, "top_k": 2048,
                          "ms": ms, "tokens_per_s": n / (ms * 1e-3), "ms_per_layer": ms / 12}), flush=True)
        del x


def static_encoder(steps=5, warmup=2, tokens=4096):
    from . import StaticSparseViTSlideEncoder, ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    net = StaticSparseViTSlideEncoder(in_features=1280, out_features=2, embed_dim=384, num_heads=6, num_layers=2,
                                      num_cls=1, window_size=3, dilation=1).to(dev).eval()
    x = torch.randn(1, tokens, 1280, generator=torch.Generator().manual_seed(1)).to(dev)

    def fwd():
        with torch.no_grad():
            return net(x)["logits"]

    ms = _time_ms(fwd, steps, warmup)
    ops.check_status(dev, "static encoder forward")
    print(json.dumps({"workload": "static_encoder_2l", "tokens": tokens, "embed_dim": 384, "heads": 6, "window": 3,
                      "dtype": "f32 in, bf16 attention", "ms": ms, "tokens_per_s": tokens / (ms * 1e-3)}), flush=True)


WORKLOADS = {"block_sparse": block_sparse_sweep, "nsa": nsa_forward, "encoder": encoder_slides,
             "static": static_encoder}
