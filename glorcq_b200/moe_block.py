"""MoE block on the sm_100a kernels.

Drop-in for the reference's ``inference.moe_block.GraphCompatibleMoeBlock``
(inference/moe_block.py:42-436): it is built from the sub-modules of a Qwen2-MoE style sparse block
(``num_experts, top_k, norm_topk_prob, gate, experts[i].{gate_proj, up_proj, down_proj},
shared_expert, shared_expert_gate``) and returns ``(hidden_states, router_logits)``.

Where the reference has three Python dispatch paths (a per-token decode loop with a host
synchronisation, a sparse loop over all experts for prefill, and a dense all-experts path for CUDA
graphs), this block makes ONE call into the C ABI (``glq_moe_forward``): routing, per-expert token
lists, the cluster-shared x.U, fused gate|up + SwiGLU, down, shared expert and the weighted combine
all run on the device with launch shapes fixed by the token count, so the same code serves eager
prefill, eager decode and graph capture, and only the routed experts' weights are read.
"""

from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.nn as nn

from . import _lib, parallel, tiled
from ._lib import FMT_T2, MoeDesc, MoeEp, Weight
from .tiled import TiledWeight


def _fuse_tiles(a: TiledWeight, b: TiledWeight) -> TiledWeight:
    """gate|up fused weight from two plain tiled weights of one shape: pair p = (tile p of a, tile p of b).
    Pure re-indexing of the already tiled buffers (load time)."""
    if (a.fmt, a.N, a.K, a.group_size, a.rank) != (b.fmt, b.N, b.K, b.group_size, b.rank):
        raise RuntimeError("gate_proj and up_proj must share format, shape, group size and rank")
    L = _lib.lib()
    f = TiledWeight(a.fmt, a.N, a.K, a.group_size, 2, a.device)
    ntiles = (a.N + 15) // 16
    bb = 512 if a.fmt == FMT_T2 else 576
    nkb = a.codes.numel() // (((ntiles + 1) // 2) * 2 * bb)

    def tiles(t):  # [pair][kb][j][bb] -> [tile][kb][bb]
        v = t.codes.view(-1, nkb, 2, bb).permute(0, 2, 1, 3).reshape(-1, nkb, bb)
        return v[:ntiles]
    f.codes.view(ntiles, nkb, 2, bb).copy_(torch.stack([tiles(a), tiles(b)], dim=2))
    if a.fmt == FMT_T2:
        f.centroids = torch.cat([a.centroids, b.centroids]).contiguous()   # one codebook per fused matrix
        f.norms.view(ntiles, 2, 16).copy_(torch.stack([a.norms.view(-1, 16)[:ntiles], b.norms.view(-1, 16)[:ntiles]], 1))
    if a.rank > 0:
        ns = (a.rank + 63) // 64
        f.sv = torch.zeros(L.glq_sv_bytes(a.N, a.rank, 2), dtype=torch.uint8, device=a.device)
        f.rank = a.rank

        def svt(t):  # [pair][slice][2][16 rows][128 B] -> [tile][slice][2048 B]
            v = t.sv.view(-1, ns, 2, 2048).permute(0, 2, 1, 3).reshape(-1, ns, 2048)
            return v[:ntiles]
        f.sv.view(ntiles, ns, 2, 2048).copy_(torch.stack([svt(a), svt(b)], dim=2))
    return f


def _table(descs: List[Weight], device) -> torch.Tensor:
    raw = b"".join(bytes(d) for d in descs)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)


_SHARED_WS_FROM = 256 << 20       # scratch sizes above this come from the per-device pool below
_BIG_WS = {}


def _shared_big_workspace(device, nbytes, ncounters):
    """Scratch and arrival counters for prompt-sized calls, one pair per device (grown on demand, never shrunk).
    The counters are zero before a call and every kernel leaves them zero."""
    key = torch.device(device).index or 0
    ws, ctr = _BIG_WS.get(key, (None, None))
    if ws is None or ws.numel() < nbytes:
        ws = None
        _BIG_WS.pop(key, None)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    if ctr is None or ctr.numel() < ncounters:
        ctr = torch.zeros(ncounters, dtype=torch.int32, device=device)
    _BIG_WS[key] = (ws, ctr)
    return ws, ctr


class GraphCompatibleMoeBlock(nn.Module):
    """Drop-in replacement for Qwen2MoeSparseMoeBlock running on the fused kernels."""

    def __init__(self, original_block):
        super().__init__()
        self.num_experts = original_block.num_experts
        self.top_k = original_block.top_k
        self.norm_topk_prob = original_block.norm_topk_prob
        self.gate = original_block.gate
        self.experts = original_block.experts
        self.shared_expert = getattr(original_block, "shared_expert", None)
        self.shared_expert_gate = getattr(original_block, "shared_expert_gate", None)
        self.graph_mode = False          # kept for the wrapper; both modes run the same device path
        self._graph_threshold = 4        # token counts up to this combine in top-k slot order
        self._built = False
        self._keep = []                  # tensors the descriptor tables point into
        self._desc: Optional[MoeDesc] = None
        self._ws = {}
        self.parallel_shared_expert = True   # shared expert on a side stream, as the reference's side-stream LoRA
        self._side = None
        self.last_selected_experts = None
        self.last_routing_weights = None
        self._ep = (0, 1, None)          # (rank, world, process group)
        self._exchange = parallel.exchange_entries
        self.peer_exchange_max_tokens = 0   # > 0: steps of up to this many tokens exchange through peer memory
        self._peers = None

    def set_expert_parallel(self, rank: int, world: int, group=None):
        """Shard the routed experts: this rank keeps experts e with e % world == rank (the other
        entries of ``experts`` may be None or unloaded).  Call before the first forward."""
        if self._built:
            raise RuntimeError("set_expert_parallel must be called before the device tables are built")
        parallel.local_experts(self.num_experts, rank, world)   # validates
        self._ep = (int(rank), int(world), group)
        return self

    # the reference hands every block the cross-layer U pool; here the pool is tiled.tiled_ut()
    def set_global_pool(self, pools, id_maps):
        self._global_pools, self._global_id_maps = pools, id_maps

    # ---- one-time device tables ---------------------------------------------------------------
    def _build(self, device):
        E = self.num_experts
        ep_rank, ep_world, _ = self._ep
        mine = parallel.local_experts(E, ep_rank, ep_world)
        if not mine:
            raise RuntimeError("this rank holds no expert (more ranks than experts)")
        lins = {e: (self.experts[e].gate_proj, self.experts[e].up_proj, self.experts[e].down_proj) for e in mine}
        for g, u, dn in lins.values():
            for lin in (g, u, dn):
                if getattr(lin, "_tiled", None) is None:
                    raise RuntimeError("every expert projection must be a GLoRCQLinear in the tiled layout "
                                       "(2/4-bit codes with group size 128/64 multiples, or 2-bit codebook)")
        g0, _, d0 = lins[mine[0]]
        H, I = g0.in_features, g0.out_features
        fmt, gs = g0._tiled.fmt, g0._tiled.group_size
        rank = g0._tiled.rank
        gate_up, down, utg, utu, utd = ([Weight() for _ in range(E)] for _ in range(5))
        rm_gu, rm_d = [0] * (2 * E), [0] * E     # row-major U^T of the persistent decode kernel
        for e, (g, u, dn) in lins.items():
            f = _fuse_tiles(g._tiled, u._tiled)
            if (f.fmt, f.group_size, f.rank, f.N, f.K) != (fmt, gs, rank, I, H) or \
                    (dn._tiled.fmt, dn._tiled.group_size, dn._tiled.rank, dn._tiled.N, dn._tiled.K) != (fmt, gs, rank, H, I):
                raise RuntimeError("all experts of a block must share format, group size, rank and shapes")
            self._keep += [f, dn._tiled]
            gate_up[e] = f.desc
            down[e] = dn._tiled.desc
            if rank > 0:
                for lin, lst in ((g, utg), (u, utu), (dn, utd)):
                    ut = tiled.tiled_ut(lin.U)
                    self._keep.append(ut)
                    lst[e] = Weight(ut.codes.data_ptr(), None, None, None, None, None, ut.N, ut.K, 0, 0)
                rms = [tiled.rowmajor_ut(lin.U) for lin in (g, u, dn)]
                self._keep += rms
                rm_gu[e], rm_gu[E + e], rm_d[e] = (t.data_ptr() for t in rms)
        d = MoeDesc()
        d.H, d.I, d.E, d.top_k = H, I, E, self.top_k
        d.rank, d.fmt, d.group_size = rank, fmt, gs
        d.norm_topk_prob = int(bool(self.norm_topk_prob))
        d.slot_order_max_tokens = self._graph_threshold
        # router (+ shared expert gate as one more row) (+ the shared expert's U_gate^T, U_up^T, so that
        # one dense product yields the logits and the shared expert's x.U)
        has_shared = self.shared_expert is not None
        if self.gate is None:
            # experts only, routing supplied per call (GLoRCQExperts): no router product
            if has_shared:
                raise RuntimeError("a block without a router cannot have a shared expert")
            d.router_rows = d.dense0_rows = d.sh_a_row = 0
            tabs = [_table(gate_up, device), _table(down, device)]
            d.gate_up, d.down = tabs[0].data_ptr(), tabs[1].data_ptr()
            if rank > 0:
                tabs += [_table(utg + utu, device), _table(utd, device)]
                d.ut_gate_up, d.ut_down = tabs[2].data_ptr(), tabs[3].data_ptr()
            self._keep += tabs
            if fmt == FMT_T2:
                d.rot_in, d.rht_in = self._rotation(g0, device)
                d.rot_mid, d.rht_mid = self._rotation(d0, device)
            self._desc = d
            self._built = True
            return
        rows = [self.gate.weight.detach().to(device=device, dtype=torch.float16)]
        if has_shared and self.shared_expert_gate is not None:
            rows.append(self.shared_expert_gate.weight.detach().to(device=device, dtype=torch.float16).reshape(1, H))
        router_rows = sum(r.shape[0] for r in rows)
        sh_rank = 0
        if has_shared:
            sg, su = self.shared_expert.gate_proj, self.shared_expert.up_proj
            if sg.SV is not None and su.SV is not None and sg.U is not None and su.U is not None:
                sh_rank = sg.U.shape[1]
        d.router_rows, d.sh_a_row = router_rows, 0
        if sh_rank > 0 and sh_rank == rank:
            pad = (-router_rows) % 16
            if pad:
                rows.append(torch.zeros(pad, H, dtype=torch.float16, device=device))
            d.sh_a_row = router_rows + pad
            rows += [sg.U.t().to(torch.float16), su.U.t().to(torch.float16)]
        router_rm = torch.cat(rows, 0).contiguous()
        router = TiledWeight.from_dense(router_rm)
        self._keep += [router, router_rm]
        d.router_t, d.dense0_rows = router.codes.data_ptr(), router.N
        d.router_rm = router_rm.data_ptr()
        if rank > 0:
            ptrs = [torch.tensor(rm_gu, dtype=torch.int64, device=device), torch.tensor(rm_d, dtype=torch.int64, device=device)]
            self._keep += ptrs
            d.ut_rm_gate_up, d.ut_rm_down = ptrs[0].data_ptr(), ptrs[1].data_ptr()
        tabs = [_table(gate_up, device), _table(down, device)]
        d.gate_up, d.down = tabs[0].data_ptr(), tabs[1].data_ptr()
        if rank > 0:
            tabs += [_table(utg + utu, device), _table(utd, device)]
            d.ut_gate_up, d.ut_down = tabs[2].data_ptr(), tabs[3].data_ptr()
        self._keep += tabs
        # rotations of the codebook format
        if fmt == FMT_T2:
            d.rot_in, d.rht_in = self._rotation(g0, device)
            d.rot_mid, d.rht_mid = self._rotation(d0, device)
        if has_shared:
            sg, su, sd = self.shared_expert.gate_proj, self.shared_expert.up_proj, self.shared_expert.down_proj
            for lin in (sg, su, sd):
                if getattr(lin, "_tiled", None) is None:
                    raise RuntimeError("the shared expert must use GLoRCQLinear projections in the tiled layout")
            f = _fuse_tiles(sg._tiled, su._tiled)
            if (f.fmt, f.group_size, f.K) != (fmt, gs, H) or f.rank not in (0, rank) or sd._tiled.rank != f.rank:
                raise RuntimeError("the shared expert must share format, group size and rank with the routed experts")
            self._keep += [f, sd._tiled]
            d.I_shared = sg.out_features
            d.sh_gate_up, d.sh_down = f.desc, sd._tiled.desc
            if f.rank > 0:
                uts = [tiled.tiled_ut(lin.U) for lin in (sg, su, sd)]
                self._keep += uts
                d.sh_ut_gate, d.sh_ut_up, d.sh_ut_down = (u.codes.data_ptr() for u in uts)
                sd_rm = tiled.rowmajor_ut(sd.U)
                self._keep.append(sd_rm)
                d.sh_ut_rm_down = sd_rm.data_ptr()
            if fmt == FMT_T2:
                d.sh_rot_mid, d.sh_rht_mid = self._rotation(sd, device)
        self._desc = d
        self._built = True

    def _rotation(self, lin, device):
        """(tiled rotation matrix, Hadamard sign vector) of a codebook-format layer: one of them is set, or
        neither when the layer has no rotation.  Sign vectors (``_rht_signs``, attached by the loader for
        rotation_type "hadamard", inference/model_builder.py:277-286) take precedence, as in the reference
        block (inference/moe_block.py:349-351)."""
        signs = getattr(lin, "_rht_signs", None)
        if signs is not None:
            sg = signs.to(device=device, dtype=torch.float32).contiguous()
            self._keep.append(sg)
            return None, sg.data_ptr()
        rc = getattr(lin, "_rotation_cache", None)
        if rc is None:
            return None, None
        Pi = rc.get_pi(lin.turbo_dim, lin.turbo_bits, lin.turbo_seed)
        key = ("pi", Pi.data_ptr())
        cache = GraphCompatibleMoeBlock._PI
        if key not in cache:
            cache[key] = TiledWeight.from_dense(Pi.to(device=device, dtype=torch.float16).contiguous())
        self._keep.append(cache[key])
        return cache[key].codes.data_ptr(), None

    _PI = {}

    def prepare(self, device, release_linear_tiles=False):
        """Build the device tables now (otherwise done on the first forward).  With
        release_linear_tiles the per-projection tiled copies of the routed experts' gate/up weights
        are dropped once they are fused (the expert modules can then no longer run on their own)."""
        if not self._built:
            self._build(torch.device(device))
        if release_linear_tiles:
            for i in parallel.local_experts(self.num_experts, self._ep[0], self._ep[1]):
                e = self.experts[i]
                e.gate_proj._tiled = e.up_proj._tiled = None
            if self.shared_expert is not None:
                self.shared_expert.gate_proj._tiled = self.shared_expert.up_proj._tiled = None
        return self

    def launches_per_call(self) -> int:
        """Kernel launches of one forward of a few tokens (affine formats; what a captured decode step holds):
        router product, routing plan, x.U of the routed gate and up clusters, fused gate|up, h.U, down, combine,
        the shared expert's gate|up, h.U and down, and with expert parallelism the exchange kernel."""
        d = self._desc
        if d is None:
            return 0
        if self.gate is not None and _lib.lib().glq_moe_uses_fused_kernel(C.byref(d), 1):
            if self._ep[1] == 1:
                return 1                                                   # the persistent kernel, combine included
            return 2 + (1 if self.peer_exchange_max_tokens > 0 else 0)    # persistent kernel, (exchange,) combine
        n = 2 + (4 if d.rank > 0 else 2) + 1
        if self.gate is None:
            n -= 1
        if d.I_shared > 0:
            n += 3 if d.sh_ut_down else 2
        if d.fmt == FMT_T2:
            n += sum(1 for r in (d.rot_in or d.rht_in, d.rot_mid or d.rht_mid, d.I_shared > 0 and (d.sh_rot_mid or d.sh_rht_mid)) if r)
        if self._ep[1] > 1 and self.peer_exchange_max_tokens > 0:
            n += 1
        return n

    # ---- forward (inference/moe_block.py:381-436) -----------------------------------------------
    def forward(self, hidden_states, top_k_index=None, top_k_weights=None, residual=None, next_norm=None):
        """(B, S, H) -> ((B, S, H), router logits).  With top_k_index / top_k_weights ((B*S, k)) the routing
        is the caller's and no logits are returned (the fused-experts adapter).

        ``next_norm = (weight or None, eps)`` folds the decoder's next steps into the combine kernel: the
        first result becomes ``residual + block output`` (``residual`` (B, S, H), optional) and a third result
        is its RMS norm times ``weight``: ((B, S, H), logits, (B, S, H))."""
        batch_size, sequence_length, hidden_dim = hidden_states.shape
        x = hidden_states.reshape(-1, hidden_dim)
        if x.dtype != torch.float16:
            x = x.half()
        x = x.contiguous()
        if not x.is_cuda:
            raise RuntimeError("GraphCompatibleMoeBlock runs on a CUDA device only (no CPU path)")
        if not self._built:
            self._build(x.device)
        d = self._desc
        n = x.shape[0]
        out = torch.empty(n, d.H, dtype=torch.float16, device=x.device)
        given = top_k_index is not None
        if given != (self.gate is None):
            raise RuntimeError("routing must be passed exactly when the block has no router")
        logits = None if given else torch.empty(n, d.E, dtype=torch.float16, device=x.device)
        if given:
            sel_in = top_k_index.to(device=x.device, dtype=torch.int32).contiguous()
            wts_in = top_k_weights.to(device=x.device, dtype=torch.float16).contiguous()
            if sel_in.shape != (n, d.top_k) or wts_in.shape != (n, d.top_k):
                raise RuntimeError(f"top_k_index / top_k_weights must have shape ({n}, {d.top_k})")
        sel = torch.empty(n, d.top_k, dtype=torch.int32, device=x.device)
        wts = torch.empty(n, d.top_k, dtype=torch.float16, device=x.device)
        normed = res2 = nw = None
        if next_norm is not None:
            nw, eps = next_norm
            normed = torch.empty(n, d.H, dtype=torch.float16, device=x.device)
            if nw is not None:
                nw = nw.to(device=x.device, dtype=torch.float16).contiguous()
            if residual is not None:
                res2 = residual.reshape(-1, hidden_dim).to(torch.float16).contiguous()
        elif residual is not None:
            raise RuntimeError("a residual is folded in only together with next_norm")
        if n > 0:
            L = _lib.lib()
            with torch.cuda.device(x.device):
                # one workspace per token count: a block's calls run one after another (it is not re-entrant across
                # streams), and a workspace made by the warm-up call must be the one a later capture finds -- an
                # allocation inside a capture would put its zero fill into the graph, once per replay
                key = n
                if key not in self._ws:
                    nbytes = L.glq_moe_workspace_bytes(C.byref(d), n)
                    nctr = L.glq_moe_counters(C.byref(d), n)
                    if nbytes > _SHARED_WS_FROM and not torch.cuda.is_current_stream_capturing():
                        # prompt-sized calls: one scratch per device for all blocks (they run one after another;
                        # a private copy per block of a 32-layer model would not fit the device)
                        ws, ctr = _shared_big_workspace(x.device, nbytes + 256, max(nctr, 1))
                    else:
                        self._ws[key] = (torch.empty(nbytes + 256, dtype=torch.uint8, device=x.device),
                                         torch.zeros(max(nctr, 1), dtype=torch.int32, device=x.device))
                if key in self._ws:
                    ws, ctr = self._ws[key]
                base = (ws.data_ptr() + 255) // 256 * 256
                aux = fork = join = None
                if self.parallel_shared_expert and d.I_shared > 0:
                    if self._side is None:
                        self._side = (torch.cuda.Stream(device=x.device), torch.cuda.Event(), torch.cuda.Event())
                    aux, fork, join = self._side[0].cuda_stream, self._side[1], self._side[2]
                    # torch creates events lazily: record once so that the handles exist
                    if not getattr(self, "_events_ready", False):
                        fork.record()
                        join.record()
                        self._events_ready = True
                    fork, join = fork.cuda_event, join.cuda_event
                ep_rank, ep_world, group = self._ep

                def call(ep):
                    if (given or normed is not None) and ep is None:
                        ep = MoeEp(0, 1, _lib.MOE_PHASE_ALL, 0, None, None, None)
                    if given:
                        ep.sel_in, ep.weight_in = sel_in.data_ptr(), wts_in.data_ptr()
                    if normed is not None:
                        ep.normed_out, ep.norm_eps = normed.data_ptr(), float(eps)
                        ep.residual = None if res2 is None else res2.data_ptr()
                        ep.norm_weight = None if nw is None else nw.data_ptr()
                    _lib.check(L.glq_moe_forward_ep(C.byref(d), x.data_ptr(), n, out.data_ptr(),
                                                    None if logits is None else logits.data_ptr(),
                                                    sel.data_ptr(), wts.data_ptr(), base,
                                                    ws.numel() - (base - ws.data_ptr()), ctr.data_ptr(), ctr.numel(),
                                                    tiled._stream_ptr(x.device), aux, fork, join,
                                                    None if ep is None else C.byref(ep)),
                               "moe_forward")
                if ep_world == 1:
                    call(None)
                else:
                    ekey = ("entries", n)
                    if ekey not in self._ws:
                        self._ws[ekey] = torch.empty(n * d.top_k, d.H, dtype=torch.float16, device=x.device)
                    entries = self._ws[ekey]
                    by_peers = 0 < n <= self.peer_exchange_max_tokens
                    ep = MoeEp(ep_rank, ep_world, _lib.MOE_PHASE_EXPERTS, _lib.MOE_EP_NO_ZERO_FILL if by_peers else 0,
                               entries.data_ptr(), None, None)
                    call(ep)
                    if by_peers:
                        # this library's exchange kernel: peer stores into every rank's buffer, then flags
                        if self._peers is None:
                            self._peers = parallel.PeerExchange.get(
                                group, x.device, self.peer_exchange_max_tokens * d.top_k, d.H)
                        px = self._peers
                        ep.phase, ep.peers = _lib.MOE_PHASE_EXCHANGE, C.pointer(px.peers)
                        call(ep)
                        ep.phase, ep.entry_out = _lib.MOE_PHASE_COMBINE, px.local_ptr
                        call(ep)
                    else:
                        self._exchange(entries, group)
                        ep.phase = _lib.MOE_PHASE_COMBINE
                        call(ep)
        self.last_selected_experts, self.last_routing_weights = sel, wts
        if normed is not None:
            return (out.reshape(batch_size, sequence_length, hidden_dim), logits,
                    normed.reshape(batch_size, sequence_length, hidden_dim))
        return out.reshape(batch_size, sequence_length, hidden_dim), logits
