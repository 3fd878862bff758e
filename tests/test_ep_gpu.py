"""Expert-parallel FP8 layer on GPUs: one rank against the fused single-GPU entry point, two virtual ranks on one
GPU (regroup / row-map kernels, exchanges emulated by slicing), and real NCCL ranks where the box has several GPUs."""
import numpy as np
import pytest
import torch

from oracle import layers as L
from tests import workloads as W
from tests.test_ep_host import run_workers

pytestmark = pytest.mark.gpu


def load_rank(m, layer, rank, local):
    for name in ("gate", "up", "down"):
        mats = getattr(layer, name)[rank * local:(rank + 1) * local]
        m.load(name, torch.from_numpy(np.stack([p for p, _ in mats])), torch.from_numpy(np.stack([s for _, s in mats])))


def test_single_rank_matches_fused_layer():
    import darask_inference_engine_b200 as D
    layer, acts = W.fp8_layer(31, 512, 256, 16, 4, 200, zipf=1.1)
    x, logits = torch.from_numpy(acts["x"]).bfloat16().cuda(), torch.from_numpy(acts["logits"]).cuda()
    fused = D.Fp8MoeLayer(512, 256, 16, 4, 200)
    load_rank(fused, layer, 0, 16)
    ref = fused.forward(x, logits)
    for exchange in ("exact", "packed"):
        ep = D.Fp8ExpertParallelMoe(512, 256, 16, 4, 200, exchange=exchange)
        load_rank(ep, layer, 0, 16)
        out = ep.forward(x, logits)
        torch.cuda.synchronize()
        assert ep.backend.device_status() == 0
        if exchange == "exact":          # same kernels, same slot-order sum: bit for bit
            assert torch.equal(out, ref)
        W.check_output(out.cpu().numpy(), L.fp8_forward(layer, acts["x"], acts["logits"])["out"])
        assert ep.rows() == (800, 800, 0)


@pytest.mark.parametrize("world,tokens", [(2, 96), (4, 33)])
def test_virtual_ranks_on_one_gpu(world, tokens):
    """All ranks' kernels run on one GPU one after the other; the two all-to-all-v steps are done by slicing."""
    import darask_inference_engine_b200 as D
    hidden, inter, experts, topk = 256, 128, 8, 2
    local = experts // world
    layer, acts = W.fp8_layer(5 + world, hidden, inter, experts, topk, tokens * world, pool=experts, zipf=1.1)
    backends, sent = [], []
    for r in range(world):
        b = D.ep.CudaFp8Backend(hidden, inter, experts, topk, world, tokens)
        load_rank(b, layer, r, local)
        x = torch.from_numpy(acts["x"][r * tokens:(r + 1) * tokens]).bfloat16().cuda()
        lg = torch.from_numpy(acts["logits"][r * tokens:(r + 1) * tokens]).cuda()
        d = b.dispatch(x, lg)
        counts = d["ranges"][:, 0].reshape(world, local).cpu().numpy()
        offs = d["ranges"][:, 1].reshape(world, local).cpu().numpy()
        backends.append(b)
        sent.append((d, counts, offs))
    y_home = [torch.zeros(tokens * topk, hidden, device="cuda") for _ in range(world)]
    for dst in range(world):                                   # what rank dst receives, in source-rank order
        recv_counts = np.stack([sent[src][1][dst] for src in range(world)]).astype(np.int32)
        pieces_c, pieces_s, origin = [], [], []
        for src in range(world):
            d, counts, offs = sent[src]
            lo, n = int(offs[dst, 0]), int(counts[dst].sum())
            pieces_c.append(d["send"][0][lo:lo + n]); pieces_s.append(d["send"][1][lo:lo + n]); origin.append((src, lo, n))
        n_recv = int(recv_counts.sum())
        pad_c = torch.zeros(128, hidden, dtype=torch.uint8, device="cuda")
        pad_s = torch.zeros(128, hidden // 128, device="cuda")
        y = backends[dst].run_experts(torch.from_numpy(recv_counts).cuda(), [torch.cat(pieces_c + [pad_c]).contiguous(),
                                                                             torch.cat(pieces_s + [pad_s]).contiguous()], n_recv)
        row = 0
        for src, lo, n in origin:                              # rows go back to where they came from
            y_home[src][lo:lo + n] = y[row:row + n]
            row += n
        assert backends[dst].device_status() == 0
    for r in range(world):
        out = backends[r].combine(y_home[r], sent[r][0]).cpu().numpy()
        ref = L.fp8_forward(layer, acts["x"][r * tokens:(r + 1) * tokens], acts["logits"][r * tokens:(r + 1) * tokens])
        assert np.array_equal(sent[r][0]["ids"].cpu().numpy(), ref["ids"])
        W.check_output(out, ref["out"])


@pytest.mark.parametrize("world,tokens", [(1, 9), (2, 40), (4, 7)])
def test_tsumuji_virtual_ranks_on_one_gpu(world, tokens):
    """The Tsumuji layer cut at its exchange steps: all ranks' kernels on one GPU, exchanges done by slicing."""
    import darask_inference_engine_b200 as D
    hidden, inter, experts, topk = 512, 256, 16, 4
    local = experts // world
    layer, acts = W.tsumuji_layer(60 + world, hidden, inter, experts, topk, tokens * world, pool=experts)
    # float32 rows that bf16 cannot hold: the hi / lo split of the window front end (more than 16 tokens) carries information
    acts["x"] = W.normal(W.rng_for(600 + world), (tokens * world, hidden), 1.0)
    t = torch.from_numpy
    backends, sent = [], []
    for r in range(world):
        b = D.ep.CudaTsumujiBackend(hidden, inter, experts, topk, world, tokens)
        b.load(t(layer.router), t(layer.blocks[r * local:(r + 1) * local].reshape(-1)), t(layer.gs[r * local:(r + 1) * local]),
               t(layer.shared_gu), t(layer.shared_down))
        d = b.dispatch(t(acts["x"][r * tokens:(r + 1) * tokens]).cuda())
        counts = d["ranges"][:, 0].reshape(world, local).cpu().numpy()
        offs = d["ranges"][:, 1].reshape(world, local).cpu().numpy()
        backends.append(b)
        sent.append((d, counts, offs))
    y_home = [torch.zeros(tokens * topk, hidden, device="cuda") for _ in range(world)]
    for dst in range(world):
        recv_counts = np.stack([sent[src][1][dst] for src in range(world)]).astype(np.int32)
        pieces, origin = [], []
        for src in range(world):
            d, counts, offs = sent[src]
            lo, n = int(offs[dst, 0]), int(counts[dst].sum())
            pieces.append(d["send"][0][lo:lo + n]); origin.append((src, lo, n))
        n_recv = int(recv_counts.sum())
        y = backends[dst].run_experts(torch.from_numpy(recv_counts).cuda(), [torch.cat(pieces).contiguous()], n_recv)
        row = 0
        for src, lo, n in origin:
            y_home[src][lo:lo + n] = y[row:row + n]
            row += n
    for r in range(world):
        out = backends[r].combine(y_home[r], sent[r][0]).cpu().numpy()
        xs = acts["x"][r * tokens:(r + 1) * tokens]
        logits = backends[r].rlogits[:tokens].cpu().numpy()
        assert np.allclose(logits, L.tsumuji_logits(layer, xs), rtol=1e-4, atol=1e-4)
        ref = L.tsumuji_forward(layer, xs, logits=logits)
        ids = sent[r][0]["ids"].cpu().numpy()
        if not np.array_equal(ids, ref["ids"]):          # only keys within 4 ulp of each other may swap (expf rounding)
            from oracle import routing as R
            keys = R.selection_keys(R.TSUMUJI, logits, layer.experts)
            for tok in np.nonzero((ids != ref["ids"]).any(1))[0]:
                a, b = keys[tok, ids[tok]], keys[tok, ref["ids"][tok]]
                assert np.all(np.abs(a - b) <= 4 * np.spacing(np.maximum(a, b)))
            ref = L.tsumuji_forward(layer, xs, logits=logits, ids=ids)
        W.check_output(out, ref["out"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tsumuji_ep_forward_nccl(tmp_path):
    world = 4 if torch.cuda.device_count() >= 4 else 2
    rows = run_workers("cuda_tsumuji", world, tmp_path, 29641)
    assert sum(r[0] for r in rows) == sum(r[1] for r in rows) and any(r[2] > 0 for r in rows)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["cuda", "cuda_exact"])          # packed slabs / exact all-to-all-v
def test_ep_forward_nccl(mode, tmp_path):
    world = min(4, torch.cuda.device_count())
    world = 2 if world == 3 else world
    rows = run_workers(mode, world, tmp_path, 29631 + (1 if mode == "cuda_exact" else 0))
    assert sum(r[0] for r in rows) == sum(r[1] for r in rows) and any(r[2] > 0 for r in rows)


@pytest.mark.parametrize("world,tokens", [(1, 50), (2, 96), (4, 33)])
def test_packed_exchange_virtual_ranks_on_one_gpu(world, tokens):
    """The exchange without sizes on the host: all ranks' kernels run on one GPU one after the other; the three equal-split
    all-to-alls are done by slicing. Outputs against the oracle, routes bit-exact."""
    import darask_inference_engine_b200 as D
    hidden, inter, experts, topk = 256, 128, 8, 2
    local = experts // world
    layer, acts = W.fp8_layer(15 + world, hidden, inter, experts, topk, tokens * world, pool=experts, zipf=1.1)
    backends, sent = [], []
    for r in range(world):
        b = D.ep.CudaFp8Backend(hidden, inter, experts, topk, world, tokens)
        load_rank(b, layer, r, local)
        x = torch.from_numpy(acts["x"][r * tokens:(r + 1) * tokens]).bfloat16().cuda()
        lg = torch.from_numpy(acts["logits"][r * tokens:(r + 1) * tokens]).cuda()
        d = b.dispatch_packed(x, lg)
        backends.append(b)
        sent.append(dict(d, send=d["send"].clone(), counts=d["counts"].clone(), ids=d["ids"].clone(), prob=d["prob"].clone()))
    zs = []
    for dst in range(world):
        recv_counts = torch.stack([sent[src]["counts"][dst] for src in range(world)]).contiguous()
        recv = torch.stack([sent[src]["send"][dst] for src in range(world)]).contiguous()
        zs.append(backends[dst].run_experts_packed(recv_counts, recv).clone())
        assert backends[dst].device_status() == 0
    for r in range(world):
        zr = torch.stack([zs[src][r] for src in range(world)]).contiguous()
        out = backends[r].sum_packed(zr, sent[r]).cpu().numpy()
        ref = L.fp8_forward(layer, acts["x"][r * tokens:(r + 1) * tokens], acts["logits"][r * tokens:(r + 1) * tokens])
        assert np.array_equal(sent[r]["ids"].cpu().numpy(), ref["ids"])
        W.check_output(out, ref["out"])


def test_packed_exchange_reports_slab_overflow():
    """A slab smaller than a destination's load: the rows that do not fit are dropped and bit 16 is set."""
    import darask_inference_engine_b200 as D
    layer, acts = W.fp8_layer(3, 256, 128, 8, 2, 64, pool=8, zipf=1.1)
    b = D.ep.CudaFp8Backend(256, 128, 8, 2, 2, 64, capacity_factor=0.25)          # 16 rows per slab, 128 routed rows
    b.dispatch_packed(torch.from_numpy(acts["x"]).bfloat16().cuda(), torch.from_numpy(acts["logits"]).cuda())
    torch.cuda.synchronize()
    assert b.device_status() & 16
    assert int(b.send_counts.sum()) == 2 * b.cap and b.cap == 16
