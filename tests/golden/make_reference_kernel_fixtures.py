"""Runs the reference's own CUDA kernels (compiled unmodified for sm_100a by
baseline/build_reference_kernels.py) on small seeded inputs and writes inputs and outputs to
tests/golden/reference_kernel_fixtures.json.  Needs a GPU:

    python baseline/build_reference_kernels.py --src <checkout of the reference>
    python tests/golden/make_reference_kernel_fixtures.py [output file]

The reference's model code is Zig and cannot be built here, but its kernels are what its model runs, so their
outputs anchor the parts of the plain implementation that its two PyTorch-made fixtures do not reach:

  head_norm   rmsnorm over each head of 128 with one gain vector (norm/norm_final.cu:28-45)
  rope        half-split pairs (i, i + 64), tables indexed by positions[t] (rope/rope_v1.cu:11-45)
  store_kv    where a token's key goes in a page: [block][kv head][slot in block][128] (attention/attention.cu:18-33)
  prefill     causal grouped-query attention of the LAST q_len positions of a longer context, over shuffled pages:
              query i sees keys 0 .. ctx - q_len + i; query head h reads kv head h // (nq / nkv) (attention.cu:300-466)
  decode      the same for the last position alone through the split kernel and its merge (attention.cu:51-207)
  sample      argmax with ties to the smaller id and the Gumbel-max draw from splitmix64 (sample/sample.cu:33-77)

bfloat16 arrays are stored as base64 of their bytes, float32 arrays as lists.  tests/test_plain.py compares the
plain functions with them.
"""
import base64
import json
import math
import os
import sys

import torch

ROOT = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
sys.path.insert(0, ROOT)


def main():
    from baseline import reference_kernels as ref
    if not ref.available() or not torch.cuda.is_available():
        print("needs a GPU and baseline/_ref (see the header)")
        return 2
    torch.manual_seed(7)
    s = ref.stream()
    torch.cuda.synchronize()
    dev = "cuda"
    nq, nkv, hd, bs = 4, 2, 128, 16
    out = {"nq": nq, "nkv": nkv, "hd": hd, "block_size": bs}

    def bf(*shape, scale=1.0):
        return (torch.randn(*shape) * scale).to(torch.bfloat16)

    def lst(t):
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            return base64.b64encode(t.view(torch.int16).numpy().tobytes()).decode("ascii")
        return t.float().flatten().tolist()

    with torch.cuda.stream(s):
        # ---- per-head norm
        eps = 1e-6
        x = bf(3, nq, hd)
        g = (1 + 0.2 * torch.randn(hd)).float()
        y = torch.empty(3, nq, hd, dtype=torch.bfloat16, device=dev)
        ref.rmsnorm(y.view(-1, hd), x.to(dev).view(-1, hd), g.to(dev), eps)
        out["head_norm"] = {"eps": eps, "x": lst(x), "gain": lst(g), "y": lst(y), "shape": [3, nq, hd]}
        # ---- rotary encoding: tables as the reference builds them (two equal halves per row), f64 angles
        theta, max_pos = 1e6, 64
        half = hd // 2
        inv = torch.tensor([1.0 / (theta ** (2.0 * i / hd)) for i in range(half)], dtype=torch.float64)
        ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
        cos = torch.cat([ang.cos(), ang.cos()], 1).float()
        sin = torch.cat([ang.sin(), ang.sin()], 1).float()
        positions = [0, 5, 37, 63]
        xr = bf(len(positions), nq, hd)
        yr = torch.empty_like(xr, device=dev)
        ref.rope(yr, xr.to(dev), cos.to(dev), sin.to(dev), torch.tensor(positions, dtype=torch.int32, device=dev), nq, hd)
        out["rope"] = {"theta": theta, "positions": positions, "x": lst(xr), "y": lst(yr), "shape": [len(positions), nq, hd]}
        # ---- store_kv: 3 tokens into slots of two different pages
        n_blocks = 4
        kc = torch.zeros(n_blocks, nkv, bs, hd, dtype=torch.bfloat16, device=dev)
        vc = torch.zeros_like(kc)
        k, v = bf(3, nkv, hd), bf(3, nkv, hd)
        slots = [2 * bs + 5, -1, 0 * bs + 15]
        ref.store_kv(k.to(dev), v.to(dev), torch.tensor(slots, dtype=torch.int32, device=dev), kc, vc, nkv, hd, bs)
        s.synchronize()
        where = kc.float().abs().sum(-1).nonzero().cpu().tolist()       # [block, kv head, slot in block] of written rows
        out["store_kv"] = {"slots": slots, "k": lst(k), "written": where, "row_2_5_head_1": lst(kc[2, 1, 5]),
                           "row_0_15_head_0_v": lst(vc[0, 0, 15])}
        # ---- attention over shuffled pages: ctx 21, the last 5 positions are this step's queries
        ctx, q_len, max_blocks, pages = 21, 5, 4, 8
        kc = bf(pages, nkv, bs, hd).to(dev)
        vc = bf(pages, nkv, bs, hd).to(dev)
        bt = [5, 2, 7, 0]
        q = bf(q_len, nq, hd)
        scale = 1.0 / math.sqrt(hd)
        o = torch.empty(q_len, nq * hd, dtype=torch.bfloat16, device=dev)
        tile = ref.attn_prefill_tile()
        q0 = list(range(0, q_len, tile))
        i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
        ref.attn_prefill(o, q.to(dev), kc, vc, i32(bt), i32([ctx]), i32([0, q_len]), i32([0] * len(q0)), i32(q0), len(q0), nq, nkv,
                         hd, max_blocks, bs, scale)
        # the keys in sequence order, for the plain function
        k_seq = torch.stack([kc[bt[t // bs], :, t % bs] for t in range(ctx)])          # [ctx, nkv, hd]
        v_seq = torch.stack([vc[bt[t // bs], :, t % bs] for t in range(ctx)])
        out["prefill"] = {"ctx": ctx, "q_len": q_len, "q": lst(q), "k_seq": lst(k_seq), "v_seq": lst(v_seq), "out": lst(o)}
        # ---- decode: the last position alone, split into parts of 8 keys and merged
        o1 = torch.empty(1, nq * hd, dtype=torch.bfloat16, device=dev)
        psize, max_parts = 8, 8
        part_o = torch.zeros(nq * max_parts * hd, dtype=torch.float32, device=dev)
        part_ml = torch.zeros(nq * max_parts * 2, dtype=torch.float32, device=dev)
        ref.attn_decode(o1, q[-1:].to(dev).contiguous(), kc, vc, i32(bt), i32([ctx]), 1, nq, nkv, hd, max_blocks, bs, scale,
                        part_o, part_ml, psize, max_parts)
        out["decode"] = {"out": lst(o1)}
        # ---- sampling: bfloat16 logits, a greedy row with a tie, two drawn rows
        V, seed = 301, 0x5EED + 0x9E3779B97F4A7C15
        logits = bf(3, V, scale=2.0)
        logits[0, 40] = logits[0, 250] = 9.0
        temps = [0.0, 0.7, 1.5]
        ids = torch.zeros(3, dtype=torch.int32, device=dev)
        scratch = torch.empty(ref.sample_scratch_bytes(3), dtype=torch.uint8, device=dev)
        ref.sample(ids, logits.to(dev), torch.tensor(temps, device=dev), torch.tensor([seed - (1 << 64) if seed >= (1 << 63) else seed], dtype=torch.int64, device=dev), scratch)
        s.synchronize()
        ref.check("fixtures")
        out["sample"] = {"V": V, "seed": seed, "temps": temps, "logits": lst(logits), "ids": ids.cpu().tolist()}
    dst = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kernel_fixtures.json")
    with open(dst, "w", encoding="utf-8") as f:
        json.dump(out, f)
    print("wrote", dst, os.path.getsize(dst), "bytes")
    return 0


if __name__ == "__main__":
    sys.exit(main())
