"""Worker of tests/test_gpu_peer.py (one process per GPU under torch.distributed.run): the
vocabulary-parallel LM head with the peer-store exchange must return the ids of the NCCL exchange
on the same inputs, over several steps, shapes and modes (so that both buffer halves, slot
padding and interleaved shapes are exercised)."""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import qx_oracle as O                      # noqa: E402  (test infrastructure)
from quixicore_metal_b200 import parallel              # noqa: E402


def main():
    rank, world, lr = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    V, K = 20000, 512
    rng = np.random.default_rng(3)
    Wq = O.synth_pack("q8_0", (0.02 * rng.standard_normal((V, K))).astype(np.float32))
    b, e = parallel.vocab_shard_bounds(V, world)[rank]
    w = torch.from_numpy(Wq[b:e]).to(dev)
    peer = parallel.VocabParallelLMHead(w, V, "q8_0", exchange="auto")
    nccl = parallel.VocabParallelLMHead(w, V, "q8_0", exchange="nccl")
    g = torch.Generator(device="cpu"); g.manual_seed(5)
    bad = 0
    for step in range(12):
        T = (1, 7, 64)[step % 3]
        mode, kw = (("argmax", {}), ("topk", {"k": 50, "temperature": 0.8}), ("topp", {"k": 32, "temperature": 0.8, "top_p": 0.9}),
                    ("categorical", {"temperature": 0.9}))[step % 4]
        h = torch.randn((T, K), generator=g).bfloat16().to(dev)
        a = peer.sample(h, mode, seed=step, **kw)
        c = nccl.sample(h, mode, seed=step, **kw)
        bad += int((a != c).sum())
    # tensor-parallel projection stack: partial sums over peer stores against NCCL all-reduce, eager and
    # replayed from a CUDA graph (the step number of the exchange is device state)
    hidden, q, kv, inter, fmt = 1024, 2048, 1024, 4096, "nvfp4"
    rs = np.random.default_rng(11)
    mk = lambda n, k: torch.from_numpy(O.synth_pack(fmt, (0.02 * rs.standard_normal((n, k))).astype(np.float32))).to(dev)
    full = {"qkv": mk(q + 2 * kv, hidden), "o": mk(hidden, q), "gate": mk(inter, hidden), "up": mk(inter, hidden),
            "down": mk(hidden, inter)}
    mine = parallel.TPDecodeStack.shard_layer(full, rank, world, fmt, q, kv)
    sp = parallel.TPDecodeStack([mine, mine], fmt, exchange="auto")
    sn = parallel.TPDecodeStack([mine, mine], fmt, exchange="nccl")
    stack_bad = 0
    for M in (1, 5):
        x = (torch.randn((M, hidden), generator=g) * 0.05).bfloat16().to(dev)
        a, c = sp.forward(x).float(), sn.forward(x).float()
        stack_bad += int(((a - c).abs() > c.abs() * 2.0 ** -6 + 1e-3 * c.abs().max()).sum())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            sp.forward(x)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y = sp.forward(x)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        stack_bad += int(((y.float() - c).abs() > c.abs() * 2.0 ** -6 + 1e-3 * c.abs().max()).sum())
    bad += stack_bad + sp.exchange_status()
    used, status = peer.exchange_used(), peer.exchange_status()
    t = torch.tensor([bad, status, 1 if used == "peer" else 0], device=dev)
    dist.all_reduce(t)
    if rank == 0:
        assert int(t[0]) == 0 and int(t[1]) == 0, t.tolist()
        print("peer exchange ok" if int(t[2]) == world else "peer exchange ok (nccl fallback: no symmetric memory)", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
