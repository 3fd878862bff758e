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
    if mode == "cuda":
        m = D.Fp8ExpertParallelMoe(HIDDEN, INTER, EXPERTS, TOPK, TOKENS_PER_RANK)
        local = EXPERTS // world
        for name in ("gate", "up", "down"):
            mats = getattr(layer, name)[rank * local:(rank + 1) * local]
            m.load(name, torch.from_numpy(np.stack([p for p, _ in mats])), torch.from_numpy(np.stack([s for _, s in mats])))
        out = m.forward(torch.from_numpy(x).bfloat16().cuda(), torch.from_numpy(logits).cuda())
        torch.cuda.synchronize()
        assert m.backend.device_status() == 0
        info, out = m.info, out.cpu().numpy()
        ids = info["ids"].cpu().numpy()
    else:
        out, info = D.ep.ep_forward(OracleBackend(layer, rank, world), torch.from_numpy(x), torch.from_numpy(logits))
        out, ids = out.numpy(), info["ids"]
    assert np.array_equal(ids, ref["ids"]), "routes differ"
    W.check_output(out, ref["out"])
    assert info["send_rows"] == TOKENS_PER_RANK * TOPK
    dist.barrier()
    with open(os.path.join(out_dir, f"ok.{rank}"), "w") as f:
        f.write(f"{info['send_rows']} {info['recv_rows']} {info['cross_rows']}\n")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
