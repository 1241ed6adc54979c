"""Secondary workloads of the sparse-attention path, timed on one GPU with CUDA events.

    python bench.py --workload dsa_variants     # DSA attention: dense sweep vs per-query row gather, one- and two-pass softmax
    python bench.py --workload block_sparse     # 2-D block-sparse sweep: H=16, D=128, block 128
    python bench.py --workload nsa              # NSA-style attention, 65536 tokens, 16 q / 2 kv heads, D=128
    python bench.py --workload encoder          # 12-layer DSA slide encoder (d=768, 12x64, top-2048) on 4 slide sizes
    python bench.py --workload static           # 2-layer static-pattern encoder (d=384, 6x64), 4096 tokens
    python bench.py --workload static2d         # 2-layer 2-D block-pattern encoder, 4096 patches on a 64x64 grid, with its CPU baseline
    torchrun ... bench.py --workload encoder --gpus N    # the ragged 4-slide batch, sequence-sharded over N GPUs

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


def synthetic_slide(n_tokens, seed, grid=512, feat=1280):
    """A synthetic slide: tissue mask = union of 3-8 seeded random ellipses on a grid x grid patch grid,
    kept cells in raster order trimmed / padded to `n_tokens`; coordinates (row, col) * 224 (level-0 pixel
    offsets, the convention of the reference's preprocessing); features N(0,1)."""
    rng = np.random.default_rng(seed)
    yy, xx = np.mgrid[0:grid, 0:grid]
    mask = np.zeros((grid, grid), dtype=bool)
    for _ in range(int(rng.integers(3, 9))):
        cy, cx = rng.uniform(0.15 * grid, 0.85 * grid, size=2)
        ay, ax = rng.uniform(0.08 * grid, 0.35 * grid, size=2)
        mask |= ((yy - cy) / ay) ** 2 + ((xx - cx) / ax) ** 2 <= 1.0
    cells = np.argwhere(mask)
    if len(cells) < n_tokens:                                   # too little tissue: add the nearest outside cells
        rest = np.argwhere(~mask)
        cells = np.concatenate([cells, rest[rng.permutation(len(rest))[: n_tokens - len(cells)]]])
        cells = cells[np.lexsort((cells[:, 1], cells[:, 0]))]
    else:
        cells = cells[np.sort(rng.permutation(len(cells))[:n_tokens])]
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_tokens, feat, generator=g).to(torch.bfloat16)
    return x, torch.from_numpy(cells.astype(np.float32) * 224.0)


def encoder_slides(steps=2, warmup=1, sizes=(24576, 57344, 98304, 131072)):
    """The full sequence-sharded encoder forward over a ragged batch: 12 x (DSA block d=768, 12 heads x 64,
    MLP 3072, top-2048, 4 x 64 indexer) with 2-D RoPE on the patch coordinates, bf16 autocast,
    random-init seeded weights; 4 synthetic slides (tissue masks on a 512 x 512 grid).  One process
    per GPU (torchrun): every slide is split over all ranks, K / V and the indexer keys are
    all-gathered per layer.  Prints one JSON line: per-slide and whole-batch time (max over ranks)."""
    import torch.distributed as dist

    from . import DSAViTSlideEncoder, ops
    from .dist import sharded_ragged_forward
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    net = DSAViTSlideEncoder(in_features=1280, out_features=2, embed_dim=768, num_heads=12, num_layers=12, num_cls=2,
                             indexer_heads=4, indexer_dim=64, top_k=2048, rope_coord_high=224.0 * 512).to(dev).eval()
    slides, coords = zip(*(synthetic_slide(n, seed=10 + i) for i, n in enumerate(sizes)))
    slides = [s.to(dev) for s in slides]
    coords = [c.to(dev) for c in coords]
    comm = torch.cuda.Stream(dev) if world > 1 else None

    def fwd(which):
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            return sharded_ragged_forward(net, [slides[i] for i in which], world, rank,
                                          coords=[coords[i] for i in which], comm_stream=comm)["logits"]

    def timed(which):
        for _ in range(warmup):
            fwd(which)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            out = fwd(which)
        b.record()
        torch.cuda.synchronize(dev)
        ms = torch.tensor([a.elapsed_time(b) / steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms[0]), out

    per_slide = [timed([i])[0] for i in range(len(sizes))]
    batch_ms, logits = timed(list(range(len(sizes))))
    ops.check_status(dev, "encoder forward")
    if rank == 0:
        total = sum(sizes)
        print(json.dumps({"workload": "dsa_encoder_12l_ragged_batch", "n_gpus": world, "slides": list(sizes),
                          "embed_dim": 768, "heads": 12, "layers": 12, "top_k": 2048, "rope": "2-D, coords (row, col) * 224",
                          "dtype": "bf16 autocast", "ms_per_slide": per_slide, "batch_ms": batch_ms,
                          "tokens_per_s": total / (batch_ms * 1e-3), "logits_finite": bool(torch.isfinite(logits).all()),
                          "parallelism": f"sp{world}" if world > 1 else "single"}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def static2d_encoder(steps=5, warmup=2, cpu_forward=None):
    """2-layer 2-D block-pattern model: 4096 patches (1280-d) on a 64 x 64 grid in 8 x 8 tiles, 1 CLS token,
    d_model 384, 6 heads x 64, Chebyshev-1 block neighbourhood + the global block, 2-D RoPE; fp32 weights,
    bf16 tensor-core attention.  `cpu_forward(state_dict, x, coords, row_ptr, col_idx) -> logits`, when
    given (bench.py passes the fp32 CPU restatement assembled from the reference's parts), is timed on
    the host cores as the CPU baseline and compared with the GPU result."""
    import time

    from . import BlockSparse2DViTSlideEncoder, ops, patterns
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    net = BlockSparse2DViTSlideEncoder(in_features=1280, out_features=2, embed_dim=384, num_heads=6, num_layers=2,
                                       num_cls=1, block=64, coord_high=64.0).eval()
    x = torch.randn(4096, 1280, generator=torch.Generator().manual_seed(1))
    t = torch.arange(4096)
    blk, tin = t // 64, t % 64
    coords = torch.stack([(blk // 8) * 8 + tin // 8, (blk % 8) * 8 + tin % 8], dim=1).float()
    rp, ci = patterns.chebyshev_grid_blocks(8, 8, 1, global_blocks=[64])
    line = {"workload": "block2d_encoder_2l", "tokens": 4096, "embed_dim": 384, "heads": 6, "block": 64,
            "pattern": "Chebyshev-1 on the 8x8 block grid + 1 global block", "dtype": "f32 weights, bf16 attention"}
    if cpu_forward is not None:
        t0 = time.perf_counter()
        ref = cpu_forward(net.state_dict(), x, coords, rp, ci)
        line["cpu_baseline"] = {"ms": (time.perf_counter() - t0) * 1e3, "cores": torch.get_num_threads(),
                                "kind": "port", "sample": "the whole forward, fp32, dense masked attention"}
    net = net.to(dev)
    xd, cd = x.to(dev), coords.to(dev)
    rpd, cid = torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev)

    def fwd():
        with torch.no_grad():
            return net(xd, cd, rpd, cid)["logits"]

    ms = _time_ms(fwd, steps, warmup)
    ops.check_status(dev, "block2d encoder forward")
    line.update({"ms": ms, "tokens_per_s": 4096 / (ms * 1e-3)})
    if cpu_forward is not None:
        line["max_abs_diff_vs_cpu"] = float((fwd()[0].cpu() - ref).abs().max())
    print(json.dumps(line), flush=True)


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


def dsa_variants(steps=3, warmup=1, sizes=(16384, 65536, 131072)):
    """The DSA attention step three ways on the same key lists (8 heads x 64, top-2048, bf16):
    `dense_sweep` = all key tiles on the tensor cores with the selection applied inside a dense softmax
    (dsa_attn_masked_kernel); `list_tiles` = the same tensor-core tiles with a sparse softmax over
    per-tile member lists (dsa_tile_lists_kernel + dsa_attn_lists_kernel); `list_gather` = the literal
    operator, every selected key / value row fetched per query and head (dsa_attn_gather_rows_kernel).
    Also the dense sweep forced onto its two-pass softmax (heavily tied indexer scores)."""
    from . import ops
    dev = torch.device("cuda", 0)
    H, D, IH, ID, K = 8, 64, 4, 64, 2048
    for T in sizes:
        g = torch.Generator().manual_seed(0)
        q = (torch.randn(1, T, H, D, generator=g) / 8).to(torch.bfloat16).to(dev).transpose(1, 2)
        k = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16).to(dev).transpose(1, 2)
        v = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16).to(dev).transpose(1, 2)
        qi = torch.randn(1, T, IH, ID, generator=g) / 8
        ki = torch.randn(1, T, IH, ID, generator=g) / 8
        w = torch.randn(IH, generator=g).to(dev)
        line = {"workload": "dsa_attention_variants", "tokens": T, "heads": H, "head_dim": D, "top_k": K}
        for tag, qq, kk in (("", qi, ki), ("_tied", (qi * 4).round() / 4, (ki * 4).round() / 4)):
            qq, kk = qq.to(torch.bfloat16).to(dev), kk.to(torch.bfloat16).to(dev)
            idx, valid, scores, sel = ops.dsa_indexer_topk(qq, kk, w, K, want_mask=True)
            o = torch.empty((1, H, T, D), dtype=torch.bfloat16, device=dev)
            line["dense_sweep" + tag + "_ms"] = _time_ms(lambda: ops.dsa_attention_masked(q, k, v, sel, o), steps, warmup)
            if tag == "":
                o3 = torch.empty_like(o)
                line["list_tiles_ms"] = _time_ms(lambda: ops.dsa_attention_lists(q, k, v, idx, scores, sel, o3), steps,
                                                 warmup)
                line["max_abs_diff_sweep_vs_list_tiles"] = float((o.float() - o3.float()).abs().max())
                if T > 65536:
                    continue            # (the row gather takes T * K time and adds nothing new beyond 65536)
                rw = scores * valid
                o2 = torch.empty_like(o)
                ms = _time_ms(lambda: ops.dsa_attention_gather(q, k, v, idx, valid, rw, o2), steps, warmup)
                gathered = 2.0 * T * K * H * D * 2
                line.update({"list_gather_ms": ms, "gathered_bytes": gathered,
                             "gather_GBps": gathered / (ms * 1e-3) / 1e9,
                             "max_abs_diff_between_variants": float((o.float() - o2.float()).abs().max())})
            del idx, valid, scores, sel
        ops.check_status(dev, "dsa variants")
        print(json.dumps(line), flush=True)


def dsa_backward(steps=3, warmup=1, sizes=(16384, 65536)):
    """The two backward operators on the bench shapes (8 heads x 64, 4 x 64 indexer, top-2048, bf16
    activations, fp32 gradients): gradients of the routing-weighted attention w.r.t. q, k, v and the
    routing weights, and of the indexer w.r.t. its projections and head weights."""
    from . import ops
    dev = torch.device("cuda", 0)
    H, D, IH, ID, K = 8, 64, 4, 64, 2048
    for T in sizes:
        g = torch.Generator().manual_seed(0)
        q = (torch.randn(1, T, H, D, generator=g) / 8).to(torch.bfloat16).to(dev).transpose(1, 2)
        k = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16).to(dev).transpose(1, 2)
        v = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16).to(dev).transpose(1, 2)
        qi = (torch.randn(1, T, IH, ID, generator=g) / 8).to(torch.bfloat16).to(dev)
        ki = (torch.randn(1, T, IH, ID, generator=g) / 8).to(torch.bfloat16).to(dev)
        w = torch.randn(IH, generator=g).to(dev)
        idx, valid, scores, sel = ops.dsa_indexer_topk(qi, ki, w, K, want_mask=True)
        o = torch.empty((1, H, T, D), dtype=torch.bfloat16, device=dev)
        ops.dsa_attention_dense(q, k, v, idx, scores, sel, o)
        d_out = torch.randn(1, T, H, D, generator=g).to(torch.bfloat16).to(dev).transpose(1, 2)
        rw = scores * valid
        ms_attn = _time_ms(lambda: ops.dsa_attention_bwd(d_out, q, k, v, o, idx, valid, rw), steps, warmup)
        d_scores = torch.randn(1, T, K, generator=g).to(dev)
        ms_idx = _time_ms(lambda: ops.dsa_indexer_bwd(d_scores, qi, ki, w, idx, valid), steps, warmup)
        ops.check_status(dev, "dsa backward")
        pairs = float(T) * min(K, T)
        print(json.dumps({"workload": "dsa_backward", "tokens": T, "heads": H, "head_dim": D, "top_k": K,
                          "attention_bwd_ms": ms_attn, "indexer_bwd_ms": ms_idx,
                          # per selected (query, key) pair and head: q, k, v, dO rows read, dk, dv rows reduced
                          "attention_bwd_gathered_GBps": pairs * H * D * (3 * 2 + 2 * 4) / (ms_attn * 1e-3) / 1e9}),
              flush=True)
        del idx, valid, scores, sel, rw, d_scores


WORKLOADS = {"dsa_backward": dsa_backward, "dsa_variants": dsa_variants, "block_sparse": block_sparse_sweep, "nsa": nsa_forward, "encoder": encoder_slides,
             "static": static_encoder, "static2d": static2d_encoder}
