"""Multi-GPU forms of the path: one process per GPU; the LM head's exchange step and the projection
stack's all-reduces of decode-sized partials run on this library's own peer-store kernels over NVLink
(symmetric allocations); torch.distributed (NCCL) is the fallback and carries large all-reduces.

Vocabulary-parallel `lm_head_sample`: the vocabulary is cut at multiples of 256 so that every
256-row tile of the reference's top-p pool lives on one GPU; each rank runs stage 1 on its rows
(ids stay global), one exchange moves the per-rank candidates ((val,id) per row for argmax /
categorical, k pairs for top-k, the tile pools and tile log-sum-exps for top-p), and every rank
runs the same stage 2.  Max-with-lowest-id, top-k-of-top-k and sum-of-exp merges are associative,
so the ids equal the single-GPU call on the same logits.  The reference has no multi-device code;
the split follows its two-stage tile -> reduce structure
(kernels/quantization/lm_head/lm_head.metal:219-235, :444-529).
"""
from __future__ import annotations

import os

import torch

from . import _lib
from .tk import _LM_HEAD_MODES, _LM_QUANT_BLOCK_K
from .tk_torch import _DT, _check, _check_lm_head, _guard, _ptr, _same_device, _stream, _workspace

TILE_V = 256


def vocab_shard_bounds(V: int, shards: int):
    """[(row_begin, row_end)] per shard: whole 256-row tiles, spread as evenly as possible."""
    tiles = (V + TILE_V - 1) // TILE_V
    base, extra = divmod(tiles, shards)
    out, t = [], 0
    for s in range(shards):
        n = base + (1 if s < extra else 0)
        out.append((min(t * TILE_V, V), min((t + n) * TILE_V, V)))
        t += n
    return out


def max_shard_tiles(V: int, shards: int) -> int:
    tiles = (V + TILE_V - 1) // TILE_V
    return max(1, -(-tiles // shards))


def _mode_id(mode) -> int:
    if isinstance(mode, str):
        if mode not in _LM_HEAD_MODES:
            raise ValueError(f"lm_head_sample: mode must be one of {list(_LM_HEAD_MODES)}")
        return _LM_HEAD_MODES[mode]
    return int(mode)


def candidate_layout(mode, k: int, max_tiles: int):
    """(C, L): candidates and tile log-sum-exps a shard emits per hidden row."""
    m = _mode_id(mode)
    kk = int(k) if int(k) > 0 else (32 if m >= 2 else 0)
    C = int(_lib.lib().qx_cuda_lm_head_shard_candidates(m, max(kk, 1), max_tiles))
    return C, (max_tiles if m == 3 else 0)


def candidate_exchange_form(per: int, world: int) -> str:
    """How slots of `per` floats cross the ranks of the peer exchange: "words" (one launch, 16-byte
    words that carry the step number: twice the bytes, no fence and no flag) while a rank sends at
    most 1 MB, else "push" (plain stores, then a flag word)."""
    stride = (per + 3) // 4 * 4
    return "words" if 8 * stride * (world - 1) <= (1 << 20) else "push"


def partial_sum_over_peers(n: int, world: int) -> bool:
    """Whether fp32 partials of n floats are summed by the one-launch peer-store all-reduce: while a
    rank sends at most 4 MB (8 bytes per float and peer); larger ones keep NCCL's algorithms."""
    return n % 2 == 0 and 8 * n * (world - 1) <= (4 << 20)


def lm_head_shard_partials(h, wq_local, bias_local, vocab_offset: int, max_tiles: int, fmt: str,
                           mode, k=0, temperature=1.0, seed=0, out=None):
    """Stage 1 on this shard's rows.  Returns one fp32 tensor (T, 2C + L) holding, per row,
    C candidate values, C candidate ids (int32 bits) and L tile log-sum-exps: a single buffer so
    that one all-gather moves everything."""
    m = _mode_id(mode)
    kk = int(k) if int(k) > 0 else (32 if m >= 2 else 0)
    if fmt not in _LM_QUANT_BLOCK_K:
        raise ValueError(f"lm_head_sample: quant format must be one of {list(_LM_QUANT_BLOCK_K)}")
    V_local = wq_local.shape[0]
    K = wq_local.shape[1] * _LM_QUANT_BLOCK_K[fmt]
    _check_lm_head(h, wq_local, bias_local, V_local, K, fmt, m, kk, float(temperature), 1.0)
    if out is not None:
        _same_device("lm_head_shard_partials", h, out)
    T = h.size(0)
    C, L = candidate_layout(m, kk, max_tiles)
    lib = _lib.lib()
    with _guard(h.device):
        hc, wc = h.contiguous(), wq_local.contiguous()
        bc = None
        if bias_local is not None and bias_local.numel() > 1:
            _check(bias_local.numel() == V_local, "lm_head_sample_q: bias must be (V,)")
            bc = bias_local.to(torch.float32).contiguous()
        # planar layout inside the buffer: [T*C vals | T*C ids | T*L lses]
        if out is None:
            out = torch.empty(T * (2 * C + L), dtype=torch.float32, device=h.device)
        val = out[: T * C]
        idt = out[T * C: 2 * T * C]
        lse = out[2 * T * C:] if L else None
        nbytes = lib.qx_cuda_lm_head_shard_workspace_bytes(T, V_local, K, m, max(kk, 1))
        ws = _workspace(h.device, nbytes)
        _lib.check(lib.qx_cuda_lm_head_shard_partials_q(
            _stream(), _ptr(hc), _ptr(wc), _ptr(bc), _ptr(val), _ptr(idt), _ptr(lse), _ptr(ws),
            nbytes, T, V_local, K, int(vocab_offset), int(max_tiles), fmt.encode(), _DT[h.dtype], m,
            max(kk, 1), float(temperature), int(seed) & 0xFFFFFFFF))
    return out


def lm_head_reduce_gathered(gathered, shards: int, T: int, max_tiles: int, mode, k=0,
                            temperature=1.0, seed=0, top_p=0.9, stride=None):
    """Stage 2 over `shards` stage-1 buffers laid end to end (the all-gather output), or `stride`
    elements apart (slots padded to a multiple of 16 bytes for the peer exchange)."""
    m = _mode_id(mode)
    kk = int(k) if int(k) > 0 else (32 if m >= 2 else 0)
    C, L = candidate_layout(m, kk, max_tiles)
    per = T * (2 * C + L)
    g = gathered.view(-1)
    with _guard(gathered.device):
        # the planar per-shard buffers are read in place: values, ids and lses start at fixed
        # offsets of shard 0 and every further shard lies `per` elements on
        base = g.data_ptr()
        ids = torch.empty(T, dtype=torch.int32, device=gathered.device)
        _lib.check(_lib.lib().qx_cuda_lm_head_shard_reduce(
            _stream(), base, base + 4 * T * C, (base + 8 * T * C) if L else None, _ptr(ids), shards, T,
            max_tiles, (int(stride) if stride else per) if shards > 1 else 0, m, max(kk, 1), float(temperature),
            int(seed) & 0xFFFFFFFF, float(top_p)))
    return ids


def lm_head_merge(parts, mode, k=0, temperature=1.0, seed=0, top_p=0.9, max_tiles=None):
    """Merge stage-1 buffers that already sit on one device (single-process form of the
    exchange, used by tests and by callers that own several shards)."""
    m = _mode_id(mode)
    kk = int(k) if int(k) > 0 else (32 if m >= 2 else 0)
    per = parts[0].numel()
    if m == 3:
        if max_tiles is None:                      # per = T*(2*mt*kk + mt): needs T; infer below
            raise ValueError("lm_head_merge: pass max_tiles for mode topp")
        T = per // (2 * max_tiles * kk + max_tiles)
    else:
        max_tiles = max_tiles or 1
        C = 1 if m <= 1 else kk
        T = per // (2 * C)
    return lm_head_reduce_gathered(torch.cat([p.reshape(-1) for p in parts]), len(parts), T,
                                   max_tiles, m, kk, temperature, seed, top_p)


class _PeerExchange:
    """Per process group: symmetric buffers by shape, the running step number, the status word."""

    def __init__(self):
        self.peer = {}
        self.step = 0
        self.status = None


class VocabParallelLMHead:
    """One rank's shard of a packed LM head plus the merge over a process group.

    wq_local holds rows [begin, end) of the full (V, K/block_k, block_bytes) matrix, where
    (begin, end) = vocab_shard_bounds(V, world)[rank].  `sample` returns the same int32 (T,)
    ids on every rank."""

    _shared = {}

    def __init__(self, wq_local, V: int, fmt: str, group=None, bias_local=None, exchange: str = "auto"):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.V, self.fmt = int(V), fmt
        # every rank must own at least one 256-row tile: an empty shard would fail its argument
        # checks while its peers already wait inside the all-gather
        tiles = (self.V + TILE_V - 1) // TILE_V
        if tiles < self.world:
            raise ValueError(f"VocabParallelLMHead: a vocabulary of {self.V} rows has {tiles} tiles of "
                             f"{TILE_V} rows, fewer than the {self.world} ranks; use fewer ranks")
        self.begin, self.end = vocab_shard_bounds(self.V, self.world)[self.rank]
        _check(wq_local.shape[0] == self.end - self.begin,
               "VocabParallelLMHead: wq_local must hold this rank's rows of vocab_shard_bounds")
        self.wq, self.bias = wq_local, bias_local
        self.max_tiles = max_shard_tiles(self.V, self.world)
        self._gather = {}
        # exchange of the per-shard candidates: "peer" = plain stores into every peer's buffer by this
        # library's own kernels (symmetric allocation), "nccl" = all_gather_into_tensor.  "auto" takes
        # the peer form when the symmetric allocation can be made and falls back to NCCL otherwise.
        self.exchange = exchange if self.world > 1 else "none"
        # Exchange buffers, the step counter and the status word belong to the process group, not to
        # one head: every head of the group uses them in the same order on every rank, so sharing keeps
        # the step numbers of all ranks aligned and costs one symmetric allocation per shape.
        self._x = VocabParallelLMHead._shared.setdefault(id(group) if group is not None else 0, _PeerExchange())
        self._head_cache = {}

    # ---- peer exchange ----------------------------------------------------------------------
    def _peer_state(self, per: int, device, shape_key=()):
        """Symmetric buffers for slots of `per` floats: two halves of world slots (padded to 16 bytes),
        either as 16-byte words that carry their step number (small slots) or as plain floats with a
        flag word per rank and the push kernel's ticket word (large slots).  None
        when the symmetric allocation is not available (every rank then takes the NCCL path: the
        decision is agreed over the group so that no rank waits for a peer that went the other way)."""
        key = (per, device) + tuple(shape_key)
        if key in self._x.peer:
            return self._x.peer[key]
        st = None
        ok = 1
        try:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            stride = (per + 3) // 4 * 4
            grp = self.group if self.group is not None else self.dist.group.WORLD
            # slots of a few KB (argmax / top-k candidates, the pools of one row) go as 16-byte words that
            # carry their own step number - one launch, one NVLink crossing; larger ones as plain
            # stores followed by a flag (half the bytes)
            if candidate_exchange_form(per, self.world) == "words":
                words = symm.empty(4 * self.world * stride, dtype=torch.float32, device=device)
                words.zero_()
                hw = symm.rendezvous(words, grp)
                st = {"stride": stride, "buf": torch.zeros(self.world * stride, dtype=torch.float32, device=device),
                      "words": words, "wptr": list(hw.buffer_ptrs), "keep": hw}
            else:
                buf = symm.empty(2 * self.world * stride, dtype=torch.float32, device=device)
                flags = symm.empty(64, dtype=torch.int32, device=device)
                buf.zero_(); flags.zero_()
                hb, hf = symm.rendezvous(buf, grp), symm.rendezvous(flags, grp)
                st = {"stride": stride, "buf": buf, "flags": flags, "bptr": list(hb.buffer_ptrs), "fptr": list(hf.buffer_ptrs),
                      "tickets": torch.zeros(1, dtype=torch.int32, device=device), "keep": (hb, hf)}
        except Exception:                                   # no symmetric memory on this system / build
            ok = 0
        agreed = torch.tensor([ok], dtype=torch.int32, device=device)
        self.dist.all_reduce(agreed, op=self.dist.ReduceOp.MIN, group=self.group)   # also orders the zero-fill before any push
        if int(agreed.item()) == 0:
            st = None
        if self._x.status is None:
            self._x.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._x.peer[key] = st
        return st

    def exchange_used(self) -> str:
        """'peer' once a call went through the peer-store exchange, else 'nccl' (or 'none' on one GPU)."""
        if self.world == 1:
            return "none"
        return "peer" if any(v is not None for v in self._x.peer.values()) else "nccl"

    def exchange_status(self) -> int:
        """0 while every bounded wait for the peers' flags has completed; 1 once one ran out (the ids
        of that call are invalid).  Synchronises the stream."""
        return 0 if self._x.status is None else int(self._x.status.item())

    def sample(self, h, mode="argmax", k=0, temperature=1.0, seed=0, top_p=0.9):
        m = _mode_id(mode)
        kk = int(k) if int(k) > 0 else (32 if m >= 2 else 0)
        T = h.size(0)
        C, L = candidate_layout(m, kk, self.max_tiles)
        per = T * (2 * C + L)
        st = self._peer_state(per, h.device, (T, m, kk)) if self.exchange in ("auto", "peer") else None
        if st is not None:
            return self._sample_peer(st, h, m, kk, T, per, temperature, seed, top_p)
        if self.exchange == "peer":
            raise RuntimeError("VocabParallelLMHead: exchange='peer' needs torch symmetric memory on every rank")
        key = (per, h.device)
        if key not in self._gather:
            self._gather[key] = torch.empty(self.world * per, dtype=torch.float32, device=h.device)
        g = self._gather[key]
        mine = g[self.rank * per:(self.rank + 1) * per]
        lm_head_shard_partials(h, self.wq, self.bias, self.begin, self.max_tiles, self.fmt, m, kk,
                               temperature, seed, out=mine)
        if self.world > 1:
            self.dist.all_gather_into_tensor(g, mine, group=self.group)
        return lm_head_reduce_gathered(g, self.world, T, self.max_tiles, m, kk, temperature, seed,
                                       top_p)

    def _sample_peer(self, st, h, m, kk, T, per, temperature, seed, top_p):
        """Stage 1 into this rank's slot, exchange of the slots (small slots: one launch whose 16-byte
        words carry the step number; large ones: push of the slot to every peer, then a bounded wait
        for the peers' flags), stage 2 - one library call, all on the current stream, no collective."""
        import ctypes
        self._x.step += 1
        step, stride, W = self._x.step, st["stride"], self.world
        par = step & 1
        if "calls" not in st and "words" in st:    # flag-in-data words: one local gather buffer, the peers' word buffers
            st["calls"] = [(st["buf"].data_ptr(), None)] * 2
            st["wrd"] = (ctypes.c_void_p * W)(*st["wptr"])
        if "calls" not in st:                      # per buffer half: local base, peers' addresses of this rank's slot
            st["calls"] = []
            for half in (0, 1):
                base = half * W * stride
                off = 4 * (base + self.rank * stride)
                st["calls"].append((st["buf"].data_ptr() + 4 * base,
                                    (ctypes.c_void_p * W)(*[p + off for p in st["bptr"]])))
            st["flg"] = (ctypes.c_void_p * W)(*st["fptr"])
        hk = (T, m, kk)
        if hk not in self._head_cache:             # this head's checked shapes, fp32 bias and workspace size
            V_local = self.wq.shape[0]
            K = self.wq.shape[1] * _LM_QUANT_BLOCK_K[self.fmt]
            _check_lm_head(h, self.wq, self.bias, V_local, K, self.fmt, m, kk, float(temperature), 1.0)
            _check(self.wq.is_contiguous(), "VocabParallelLMHead: wq_local must be contiguous")
            bias = None
            if self.bias is not None and self.bias.numel() > 1:
                _check(self.bias.numel() == V_local, "lm_head_sample_q: bias must be (V,)")
                bias = self.bias.to(torch.float32).contiguous()
            self._head_cache[hk] = (V_local, K, bias,
                                    _lib.lib().qx_cuda_lm_head_shard_workspace_bytes(T, V_local, K, m, max(kk, 1)))
        _check(h.is_cuda and h.dim() == 2 and h.dtype in _DT, "lm_head_sample_q: inputs must be CUDA and h must be floating point")
        _same_device("lm_head_sample_q", h, self.wq)
        V_local, K, bias32, ws_bytes = self._head_cache[hk]
        _check(h.size(1) == K and temperature > 0.0, "lm_head_sample_q: h must be (T, K), temperature positive")
        base, dst = st["calls"][par]
        with _guard(h.device):
            hc = h.contiguous()
            ws = _workspace(h.device, ws_bytes)
            ids = torch.empty(T, dtype=torch.int32, device=h.device)
            _lib.check(_lib.lib().qx_cuda_lm_head_sample_sharded(
                _stream(), hc.data_ptr(), self.wq.data_ptr(), _ptr(bias32), ids.data_ptr(), base, stride, dst,
                st.get("flg"), _ptr(st.get("flags")), _ptr(st.get("tickets")), st.get("wrd"), self._x.status.data_ptr(), W, self.rank,
                step, 5000, ws.data_ptr(), ws_bytes, T, V_local, K, self.begin, self.max_tiles,
                self.fmt.encode(), _DT[h.dtype], m, max(kk, 1), float(temperature), int(seed) & 0xFFFFFFFF,
                float(top_p)))
        return ids


# ----------------------------------------------------------------------------------------------
# Tensor-parallel decode projection stack (Llama-style blocks without attention math).
# ----------------------------------------------------------------------------------------------
class TPDecodeStack:
    """Per-rank shard of a stack of decoder-block projections over packed weights.

    Per layer: QKV (column-parallel: output rows split), O (row-parallel: K split, fp32 partials
    summed by one all-reduce, then the residual is added once), fused gate/up SwiGLU
    (column-parallel), down (row-parallel + all-reduce + residual).  Attention itself is outside
    this path and is replaced by the identity on V: every local query head takes the value vector
    of its KV group, which makes the local input of O exactly this rank's K-shard.

    `layers` is a list of dicts with this rank's packed tensors:
        qkv  (q_local + 2*kv_local, hidden/bk, bb)     o    (hidden, q_local/bk, bb)
        gate (inter_local, hidden/bk, bb)  up (same)   down (hidden, inter_local/bk, bb)
    Partial sums cross the ranks in fp32 (not in the 16-bit I/O type), so the only difference from
    the single-device result is the order of the K summation."""

    def __init__(self, layers, fmt: str, head_dim: int = 128, group=None, tensor_parallel: bool = True,
                 exchange: str = "auto"):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        # tensor_parallel=False: `layers` are whole (unsharded) tensors and no collective runs, even
        # inside an initialised process group (the single-device result the sharded one is checked against)
        self.world = dist.get_world_size(group) if (tensor_parallel and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if (tensor_parallel and dist.is_initialized()) else 0
        # "auto": row-parallel partials are summed over peer stores by this library's kernels when a
        # symmetric allocation can be made, else by NCCL all-reduce; "nccl" forces the latter
        self.exchange = exchange
        self._sum = {}
        self.layers, self.fmt, self.head_dim = layers, fmt, head_dim
        bk = _LM_QUANT_BLOCK_K[fmt]
        l0 = layers[0]
        self.q_local = l0["o"].shape[1] * bk
        self.kv_local = (l0["qkv"].shape[0] - self.q_local) // 2
        _check(self.q_local % self.kv_local == 0 and self.kv_local % head_dim == 0,
               "TPDecodeStack: query width must be a multiple of the KV width, KV width of head_dim")

    def _all_reduce(self, t):
        if self.world > 1:
            self.dist.all_reduce(t, group=self.group)
        return t

    # ---- sum of the row-parallel partials over peer stores, residual add and cast fused ----------
    def _peer_sum_state(self, n: int, device):
        """Symmetric buffer (two halves of world slots of n / 2 16-byte words {x, step, y, step}), step
        counter, tickets and status for partials of n floats; None when symmetric memory is
        unavailable (agreed over the group, every rank then uses the NCCL all-reduce)."""
        key = (n, device)
        if key in self._sum:
            return self._sum[key]
        st, ok = None, 1
        try:
            import ctypes
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            buf = symm.empty(4 * self.world * n, dtype=torch.float32, device=device)
            buf.zero_()
            grp = self.group if self.group is not None else self.dist.group.WORLD
            hb = symm.rendezvous(buf, grp)
            W = self.world
            st = {"buf": buf, "keep": hb, "bptr": (ctypes.c_void_p * W)(*list(hb.buffer_ptrs)),
                  "counter": torch.zeros(1, dtype=torch.int32, device=device),
                  "tickets": torch.zeros(1, dtype=torch.int32, device=device),
                  "status": torch.zeros(1, dtype=torch.int32, device=device)}
        except Exception:
            ok = 0
        agreed = torch.tensor([ok], dtype=torch.int32, device=device)
        self.dist.all_reduce(agreed, op=self.dist.ReduceOp.MIN, group=self.group)
        if int(agreed.item()) == 0:
            st = None
        self._sum[key] = st
        return st

    def _sum_add_residual(self, part, x):
        """x + sum over the ranks of `part` (fp32 partial of this rank), in x's dtype."""
        if self.world == 1:
            return (part + x.float()).to(x.dtype)
        n = part.numel()
        # decode-sized partials are latency-bound: one-shot peer stores while a rank sends at most 4 MB
        # (8 bytes per float and peer); larger ones keep NCCL's bandwidth-optimal algorithms
        small = partial_sum_over_peers(n, self.world) or (self.exchange == "peer" and n % 2 == 0)
        st = self._peer_sum_state(n, part.device) if (self.exchange in ("auto", "peer") and small) else None
        self._last = "nccl" if st is None else "peer"
        if st is None:
            return (self._all_reduce(part) + x.float()).to(x.dtype)
        from . import _lib
        L = _lib.lib()
        pc, xc = part.contiguous(), x.contiguous()
        out = torch.empty_like(xc)
        stream = _stream()
        _lib.check(L.qx_cuda_peer_allreduce(stream, pc.data_ptr(), xc.data_ptr(), out.data_ptr(), n, st["bptr"],
                                            self.world, self.rank, st["counter"].data_ptr(), st["tickets"].data_ptr(),
                                            st["status"].data_ptr(), _DT[x.dtype], 5000))
        return out

    def exchange_used(self) -> str:
        """How the most recent partial sum crossed the ranks: 'peer', 'nccl', or 'none' on one GPU."""
        return "none" if self.world == 1 else getattr(self, "_last", "nccl")

    def exchange_status(self) -> int:
        """Number of shapes whose bounded wait for the peers ran out (their results are invalid)."""
        return sum(int(v["status"].item()) for v in self._sum.values() if v is not None)

    def layer(self, x, L, trace=None):
        """One block.  `trace`, if given, is a dict that receives the residual stream after the
        O projection ("h"), for tests that compare each half of the block on its own inputs."""
        from . import tk, tk_torch
        qkv = tk.decode_linear_epilogue(x, L["qkv"], format=self.fmt)
        # identity on V: the G query heads of KV group g all take that group's value vector
        hd = self.head_dim
        n_kv = self.kv_local // hd
        v = qkv[:, self.q_local + self.kv_local:].reshape(-1, n_kv, 1, hd)
        attn = v.expand(-1, n_kv, self.q_local // self.kv_local, hd).reshape(-1, self.q_local).contiguous()
        x = self._sum_add_residual(tk_torch.decode_linear_partial(attn, L["o"], self.fmt), x)
        if trace is not None:
            trace["h"] = x
        mid = tk.decode_swiglu(x, L["gate"], L["up"], format=self.fmt)
        return self._sum_add_residual(tk_torch.decode_linear_partial(mid, L["down"], self.fmt), x)

    def forward(self, x):
        for L in self.layers:
            x = self.layer(x, L)
        return x

    @staticmethod
    def shard_layer(full, rank: int, world: int, fmt: str, q: int, kv: int):
        """This rank's tensors cut from one layer's full packed tensors (host or device): rows of
        q / k / v / gate / up, K-blocks of o / down.  KV groups stay whole: kv % world == 0."""
        bk = _LM_QUANT_BLOCK_K[fmt]
        ql, kl = q // world, kv // world
        W = full["qkv"]
        qkv = torch.cat([W[rank * ql:(rank + 1) * ql], W[q + rank * kl:q + (rank + 1) * kl],
                         W[q + kv + rank * kl:q + kv + (rank + 1) * kl]]) if torch.is_tensor(W) else None
        il = full["gate"].shape[0] // world
        cut = lambda t, n: t[:, rank * n:(rank + 1) * n].contiguous()
        return {"qkv": qkv.contiguous(), "o": cut(full["o"], ql // bk),
                "gate": full["gate"][rank * il:(rank + 1) * il].contiguous(),
                "up": full["up"][rank * il:(rank + 1) * il].contiguous(),
                "down": cut(full["down"], il // bk)}

    def weight_bytes(self) -> int:
        return sum(t.numel() for L in self.layers for t in L.values())
