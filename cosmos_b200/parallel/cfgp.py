"""CFG parallelism: the cond and uncond guidance branches run on two rank groups at the same
time (reference: `--cfgp-size`, evaluation/cosmos3/Physics_IQ/run_with_cosmos_framework.ipynb:645;
`--cfg-parallel-size 2`, README.md:318).

Each rank computes the velocity of its own branch for its token shard. In the fused path the
branch result is written into a double-buffered symmetric buffer, one device-side barrier orders
the pair, and the CFG-combine + Euler kernel reads the other branch straight from the peer's
memory with P2P loads (no collective call, no extra copy of the peer's data). The baseline path
all-gathers the two velocities with NCCL/gloo.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist

from .mesh import Mesh
from .symm import symm_group


class CFGParallel:
    def __init__(self, mesh: Mesh, fused: bool = True):
        self.group = mesh.group("cfgp")
        self.ranks = mesh.group_ranks["cfgp"]
        assert len(self.ranks) == 2, "CFG parallelism uses exactly two branches"
        self.branch = mesh.index("cfgp")  # 0 = cond, 1 = uncond
        self.fused = bool(fused) and torch.cuda.is_available()
        self.sg = None
        self._buf = None
        self._step = 0

    def _buffers(self, like: torch.Tensor):
        if self._buf is None or self._buf[1] != tuple(like.shape):
            dev = like.device
            self.sg = symm_group(self.group, self.ranks, dev)
            nbytes = like.numel() * like.element_size()
            nb = (nbytes + 255) // 256 * 256
            buf = self.sg.alloc(f"cfgp_v_{tuple(like.shape)}_{like.dtype}", 2 * nb)
            views = []
            for slot in range(2):
                mine = buf.view(slot * nb, tuple(like.shape), like.dtype)
                peer = buf._handle.get_buffer(1 - self.branch, tuple(like.shape), like.dtype,
                                              slot * nb // like.element_size())
                views.append((mine, peer))
            self._buf = (views, tuple(like.shape))
        return self._buf[0]

    def branch_velocities(self, engine, xin: torch.Tensor, sigma: float, st, control_scale: float = 0.0,
                          guidance: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
        """Returns (v_cond, v_uncond) for this rank's token shard; one of the two lives on the peer. With a control
        stream (`control_scale` != 0) the cond branch also evaluates the prompt with the control tokens and
        publishes v_c + (g_c / g) (v_ctrl - v_c), which turns the two-branch combine into the three-branch one."""
        kv = st.ar_kv_cond if self.branch == 0 else st.ar_kv_uncond
        mdt = engine.model.patch_in.dtype
        sig = torch.full((1,), float(sigma), device=xin.device)
        v = engine.velocity(xin.to(mdt), sig, st, kv)
        if control_scale != 0.0 and self.branch == 0:
            v_ctrl = engine.velocity(xin.to(mdt), sig, st, kv, with_control=True)
            v = torch.lerp(v.float(), v_ctrl.float(), control_scale / float(guidance)).to(v.dtype)
        if self.fused and v.is_cuda:
            views = self._buffers(v)
            mine, peer = views[self._step & 1]
            self._step += 1
            mine.copy_(v)
            self.sg.barrier(slot=2)
            return (mine, peer) if self.branch == 0 else (peer, mine)
        both = [torch.empty_like(v), torch.empty_like(v)]
        dist.all_gather(both, v.contiguous(), group=self.group)
        return both[0], both[1]
