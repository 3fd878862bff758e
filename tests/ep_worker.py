"""One rank of the expert-parallel layer test; launched by tests/test_ep_*.py as

    python -m torch.distributed.run --nproc-per-node N tests/ep_worker.py {cpu|cuda} OUT_DIR

`cpu`: gloo + a numpy backend built from the oracle (checks the exchange logic of `ep_forward`);
`cuda`: NCCL + the CUDA backend.  Every rank compares its tokens' outputs with the single-process oracle.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import formats as F  # noqa: E402
from oracle import layers as L  # noqa: E402
from oracle import routing as R  # noqa: E402
from tests import workloads as W  # noqa: E402

HIDDEN, INTER, EXPERTS, TOPK, TOKENS_PER_RANK = 256, 128, 8, 2, 24


class OracleBackend:
    """numpy stand-in for the kernels of one rank (restates what each C entry point produces)."""
    pad_rows = 0

    def __init__(self, layer, rank, world):
        self.layer, self.rank, self.world = layer, rank, world
        self.local = layer.experts // world

    def dispatch(self, x, logits):
        x, logits = x.numpy(), logits.numpy()
        ids, prob = R.route_kogarashi(logits, self.layer.topk)
        assign, counts, offsets = R.permutation(ids, self.layer.experts, self.layer.topk)
        xq, xs = F.fp8_act_quantize(x)
        tok = assign.astype(np.int64) // self.layer.topk
        position = np.empty(assign.size, np.int32)
        position[assign.astype(np.int64)] = np.arange(assign.size, dtype=np.int32)
        return dict(send=[torch.from_numpy(xq[tok]), torch.from_numpy(xs[tok])],
                    ranges=torch.from_numpy(np.stack([counts, offsets], 1).astype(np.int32)), position=position, ids=ids, prob=prob,
                    tokens=x.shape[0])

    def run_experts(self, recv_counts, received, n_recv):
        counts = recv_counts.numpy().reshape(self.world, self.local)
        codes, scales = received[0].numpy(), received[1].numpy()
        y = np.zeros((n_recv, self.layer.hidden), np.float32)
        row = 0
        for r in range(self.world):
            for e in range(self.local):
                c = int(counts[r, e])
                if c:
                    ge = self.rank * self.local + e
                    g = L.fp8_dequant_gemm(codes[row:row + c], scales[row:row + c], *self.layer.gate[ge])
                    u = L.fp8_dequant_gemm(codes[row:row + c], scales[row:row + c], *self.layer.up[ge])
                    hq, hs = F.fp8_act_quantize(F.bf16_round((g / (1.0 + np.exp(-g)) * u).astype(np.float32)))
                    y[row:row + c] = L.fp8_dequant_gemm(hq, hs, *self.layer.down[ge]).astype(np.float32)
                row += c
        return torch.from_numpy(y)

    # ---- the exchange without sizes on the host: slabs of fixed capacity out, rows pre-reduced per (token, rank) back ----
    def dispatch_packed(self, x, logits):
        d = self.dispatch(x, logits)
        k, t = self.layer.topk, x.shape[0]
        cap, h = t * k, self.layer.hidden
        codes, scales = d["send"][0].numpy(), d["send"][1].numpy()
        counts = d["ranges"][:, 0].numpy().reshape(self.world, self.local)
        order = np.argsort(d["position"])                      # dispatch row -> assignment
        slabs = np.zeros((self.world, cap, h + 4 * (h // 128) + 8), np.uint8)
        row = 0
        for r in range(self.world):
            n = int(counts[r].sum())
            for j in range(n):
                a = int(order[row + j])
                slabs[r, j, :h] = codes[row + j]
                slabs[r, j, h:h + 4 * (h // 128)] = scales[row + j].view(np.uint8)
                slabs[r, j, h + 4 * (h // 128):] = np.concatenate([np.array([d["prob"][a // k, a % k]], np.float32).view(np.uint8),
                                                                    np.array([a // k], np.int32).view(np.uint8)])
            row += n
        return dict(send=torch.from_numpy(slabs), counts=torch.from_numpy(counts.astype(np.int32)), ids=d["ids"], prob=d["prob"], tokens=t)

    def run_experts_packed(self, recv_counts, recv):
        counts, slabs = recv_counts.numpy(), recv.numpy()
        h, tcap = self.layer.hidden, slabs.shape[1] // self.layer.topk
        z = np.zeros((self.world, tcap, h), np.float32)
        for s in range(self.world):
            n = int(counts[s].sum())
            rows = slabs[s, :n]
            codes = np.ascontiguousarray(rows[:, :h])
            scales = np.ascontiguousarray(rows[:, h:h + 4 * (h // 128)]).view(np.float32)
            meta = np.ascontiguousarray(rows[:, h + 4 * (h // 128):])
            prob, tok = meta[:, :4].copy().view(np.float32)[:, 0], meta[:, 4:8].copy().view(np.int32)[:, 0]
            y = self.run_experts(torch.from_numpy(np.stack([counts[s]] + [np.zeros_like(counts[s])] * (self.world - 1))), [torch.from_numpy(codes),
                                 torch.from_numpy(scales)], n).numpy() if n else np.zeros((0, h), np.float32)
            # run_experts walks (rank, expert) segments in order: with the other ranks' counts zero it is this slab alone
            for j in range(n):
                z[s, tok[j]] += prob[j] * y[j]
        return torch.from_numpy(z)

    def sum_packed(self, zr, d):
        return torch.from_numpy(zr.numpy()[:, :d["tokens"]].sum(0).astype(np.float32))

    def combine(self, y_home, d):
        y, k = y_home.numpy(), self.layer.topk
        out = np.zeros((d["tokens"], self.layer.hidden), np.float32)
        for t in range(d["tokens"]):
            for s in range(k):
                out[t] += np.float32(d["prob"][t, s]) * y[d["position"][t * k + s]]
        return torch.from_numpy(out)


def main():
    mode, out_dir = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if mode.startswith("cuda"):
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    else:
        dist.init_process_group("gloo")
    layer, acts = W.fp8_layer(77, HIDDEN, INTER, EXPERTS, TOPK, TOKENS_PER_RANK * world, pool=EXPERTS, zipf=1.1)
    lo, hi = rank * TOKENS_PER_RANK, (rank + 1) * TOKENS_PER_RANK
    x, logits = acts["x"][lo:hi], acts["logits"][lo:hi]
    ref = L.fp8_forward(layer, x, logits)
    import darask_inference_engine_b200 as D
    if mode == "cuda_tsumuji":
        tl, ta = W.tsumuji_layer(78, 512, 256, 16, 4, TOKENS_PER_RANK * world, pool=16)
        tx = ta["x"][lo:hi]
        local = 16 // world
        m = D.TsumujiExpertParallelMoe(512, 256, 16, 4, TOKENS_PER_RANK)
        t = torch.from_numpy
        m.load(t(tl.router), t(tl.blocks[rank * local:(rank + 1) * local].reshape(-1)), t(tl.gs[rank * local:(rank + 1) * local]),
               t(tl.shared_gu), t(tl.shared_down))
        out = m.forward(t(tx).cuda())
        torch.cuda.synchronize()
        tref = L.tsumuji_forward(tl, tx, logits=m.backend.rlogits[:TOKENS_PER_RANK].cpu().numpy())
        assert np.array_equal(m.info["ids"].cpu().numpy(), tref["ids"]), "routes differ"
        W.check_output(out.cpu().numpy(), tref["out"])
        info = m.info
        dist.barrier()
        with open(os.path.join(out_dir, f"ok.{rank}"), "w") as f:
            f.write(f"{info['send_rows']} {info['recv_rows']} {info['cross_rows']}\n")
        dist.destroy_process_group()
        return
    if mode in ("cuda", "cuda_exact"):
        m = D.Fp8ExpertParallelMoe(HIDDEN, INTER, EXPERTS, TOPK, TOKENS_PER_RANK, exchange="exact" if mode == "cuda_exact" else "packed")
        local = EXPERTS // world
        for name in ("gate", "up", "down"):
            mats = getattr(layer, name)[rank * local:(rank + 1) * local]
            m.load(name, torch.from_numpy(np.stack([p for p, _ in mats])), torch.from_numpy(np.stack([s for _, s in mats])))
        out = m.forward(torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(logits).cuda())
        torch.cuda.synchronize()
        assert m.backend.device_status() == 0
        out = out.cpu().numpy()
        ids = m.info["ids"].cpu().numpy()
        rows = m.rows()
    elif mode == "cpu_packed":
        out, info = D.ep.ep_forward_packed(OracleBackend(layer, rank, world), torch.from_numpy(x), torch.from_numpy(logits))
        out, ids = out.numpy(), info["ids"]
        sent = info["send_counts"].numpy().sum(1)
        rows = (int(sent.sum()), int(info["recv_counts"].numpy().sum()), int(sent.sum() - sent[rank]))
    else:
        out, info = D.ep.ep_forward(OracleBackend(layer, rank, world), torch.from_numpy(x), torch.from_numpy(logits))
        out, ids = out.numpy(), info["ids"]
        rows = (info["send_rows"], info["recv_rows"], info["cross_rows"])
    assert np.array_equal(ids, ref["ids"]), "routes differ"
    W.check_output(out, ref["out"])
    assert rows[0] == TOKENS_PER_RANK * TOPK
    dist.barrier()
    with open(os.path.join(out_dir, f"ok.{rank}"), "w") as f:
        f.write(f"{rows[0]} {rows[1]} {rows[2]}\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
