"""Shared builders for the tests: random problems, the global fp32 oracle, virtual-cluster runners."""
import torch

from teramoe_b200.engine import EPEngine
from teramoe_b200.parallel.world import VirtualCluster
from teramoe_b200.reference import moe_reference


def make_problem(N, T, H, I, E, K, seed=0, dtype=torch.float32, device="cpu", x_scale=1.0, w_scale=0.02, drop_some=False,
                 empty_expert=None, uneven_tokens=False):
    g = torch.Generator().manual_seed(seed)
    prob = {"N": N, "H": H, "I": I, "E": E, "K": K, "ranks": []}
    prob["W_gateup"] = (torch.randn(E, 2 * I, H, generator=g) * w_scale).to(dtype).to(device)
    prob["W_down"] = (torch.randn(E, H, I, generator=g) * w_scale).to(dtype).to(device)
    for r in range(N):
        Tr = T if not uneven_tokens else max(0, T - 37 * r)
        x = (torch.randn(Tr, H, generator=g) * x_scale).to(dtype)
        logits = torch.randn(Tr, E, generator=g)
        if empty_expert is not None:
            logits[:, empty_expert] = -1e9
        top = torch.topk(logits, K, dim=1)
        idx = top.indices.to(torch.int64)
        w = torch.softmax(top.values, dim=1).float()
        if drop_some and Tr > 3:
            idx[1, 0] = -1
            idx[3, K - 1] = -1
        go = torch.randn(Tr, H, generator=g).to(dtype)
        prob["ranks"].append({"x": x.to(device), "idx": idx.to(device), "w": w.to(device), "go": go.to(device)})
    return prob


def oracle(prob):
    """fp32 reference over the concatenated tokens of all ranks."""
    xs = torch.cat([r["x"] for r in prob["ranks"]]).detach().float().cpu().clone().requires_grad_(True)
    idx = torch.cat([r["idx"] for r in prob["ranks"]]).cpu()
    w = torch.cat([r["w"] for r in prob["ranks"]]).detach().float().cpu().clone().requires_grad_(True)
    Wg = prob["W_gateup"].detach().float().cpu().clone().requires_grad_(True)
    Wd = prob["W_down"].detach().float().cpu().clone().requires_grad_(True)
    go = torch.cat([r["go"] for r in prob["ranks"]]).float().cpu()
    out = moe_reference(xs, idx, w, Wg, Wd)
    out.backward(go)
    sizes = [r["x"].shape[0] for r in prob["ranks"]]
    El = prob["E"] // prob["N"]
    res = []
    outs, dxs, dws = out.detach().split(sizes), xs.grad.split(sizes), w.grad.split(sizes)
    for r in range(prob["N"]):
        res.append({"out": outs[r], "dx": dxs[r], "dw": dws[r], "dWg": Wg.grad[r * El:(r + 1) * El], "dWd": Wd.grad[r * El:(r + 1) * El]})
    return res


def run_virtual(prob, device):
    """Forward + backward of every rank of a VirtualCluster; returns per-rank dicts like oracle()."""
    N, E = prob["N"], prob["E"]
    El = E // N
    cluster = VirtualCluster(N, device)
    try:
        engines = [EPEngine(w) for w in cluster.worlds]
        Wg = [prob["W_gateup"][r * El:(r + 1) * El].contiguous() for r in range(N)]
        Wd = [prob["W_down"][r * El:(r + 1) * El].contiguous() for r in range(N)]
        fw = cluster.drive([engines[r].forward_gen(prob["ranks"][r]["x"], prob["ranks"][r]["idx"], prob["ranks"][r]["w"], Wg[r], Wd[r], E)
                            for r in range(N)])
        bw = cluster.drive([engines[r].backward_gen(fw[r][1], prob["ranks"][r]["go"], Wg[r], Wd[r]) for r in range(N)])
        if torch.device(device).type == "cuda":
            torch.cuda.synchronize()
        res = []
        for r in range(N):
            dx, gtw, dWg, dWd = bw[r]
            res.append({"out": fw[r][0], "dx": dx, "dw": gtw, "dWg": dWg, "dWd": dWd, "saved": fw[r][1]})
        return res
    finally:
        cluster.close()


def compare(res, ref, atol, rtol, names=("out", "dx", "dw", "dWg", "dWd")):
    for r, (a, b) in enumerate(zip(res, ref)):
        for n in names:
            x, y = a[n].float().cpu(), b[n].float().cpu()
            assert x.shape == y.shape, (n, x.shape, y.shape)
            if x.numel() == 0:
                continue
            err = (x - y).abs().max().item()
            lim = atol + rtol * y.abs().max().item()
            assert err <= lim, f"rank {r} {n}: max err {err} > {lim}"
