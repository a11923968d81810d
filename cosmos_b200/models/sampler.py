"""Flow-matching samplers: shifted sigma schedule, Euler and UniPC (order 2) updates, and
classifier-free guidance with the reference's knobs (`guidance`, `guidance_interval`,
`normalize_cfg`, `control_guidance`; reference evaluation/cosmos3/Physics_IQ/
run_with_cosmos_framework.ipynb:460-523 and cookbooks/cosmos3/generator/transfer/specs/edge.json:17-18;
`flow_shift` / UniPC: README.md:247).

Convention: x_sigma = (1 - sigma) * x0 + sigma * eps, sigma in [0, 1]; the network predicts the
velocity v = eps - x0, so dx/dsigma = v and one Euler step is x += (sigma_next - sigma) * v.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from .. import ops


def shifted_sigmas(num_steps: int, shift: float = 1.0, sigma_max: Optional[float] = None,
                   device=None) -> torch.Tensor:
    """num_steps+1 sigmas from 1 (or the sigma_max-derived start) to 0, warped by
    sigma' = shift*sigma / (1 + (shift-1)*sigma). `sigma_max` is an EDM-style noise level;
    it maps to the flow time sigma_max / (1 + sigma_max) (80 -> 0.9877)."""
    start = 1.0 if sigma_max is None else sigma_max / (1.0 + sigma_max)
    s = torch.linspace(start, 0.0, num_steps + 1, dtype=torch.float64, device=device)
    s = shift * s / (1.0 + (shift - 1.0) * s)
    return s.float()


def logit_normal_t(n: int, mean: float = 0.0, std: float = 1.0, generator=None, device=None) -> torch.Tensor:
    """Training timestep distribution: sigmoid(N(mean, std))."""
    return torch.sigmoid(torch.randn(n, generator=generator, device=device) * std + mean)


def guidance_active(sigma: float, interval: Sequence[float]) -> bool:
    """CFG is applied while the timestep (sigma * 1000) lies inside `guidance_interval`."""
    t = float(sigma) * 1000.0
    return interval[0] <= t <= interval[1]


def cfg_velocity(v_cond, v_uncond, guidance: float, normalize: bool = False,
                 v_control=None, control_guidance: Optional[float] = None):
    """v = v_u + g (v_c - v_u) [+ g_ctrl (v_ctrl - v_c)], optionally renormalised row-wise."""
    if v_uncond is None:
        v = v_cond.float()
    else:
        v = ops.ref.cfg_combine(v_cond, v_uncond, guidance, normalize)
    if v_control is not None and control_guidance is not None:
        v = v + control_guidance * (v_control.float() - v_cond.float())
    return v


class EulerSampler:
    def __init__(self, sigmas: torch.Tensor):
        self.sigmas = sigmas
        self.i = 0

    def step(self, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        dt = float(self.sigmas[self.i + 1] - self.sigmas[self.i])
        self.i += 1
        return x + dt * v.to(x.dtype)

    def dt(self) -> float:
        return float(self.sigmas[self.i + 1] - self.sigmas[self.i])


class UniPCSampler:
    """UniPC (B(h) = expm1(h) variant) in data-prediction form for flow sigmas, predictor order
    up to 2 with the corrector applied from the second step on.

    With alpha = 1 - sigma and lambda = log(alpha / sigma), the exact solution of the
    data-prediction ODE over a step h = lambda_next - lambda is
        x_next = (sigma_next / sigma) x - alpha_next * expm1(-h) * x0_hat  (+ higher-order terms)
    and the multistep terms use differences of the stored x0 predictions."""

    def __init__(self, sigmas: torch.Tensor, order: int = 2):
        self.sigmas = sigmas.double()
        self.order = order
        self.i = 0
        self.x0_hist: List[torch.Tensor] = []
        self.lam_hist: List[float] = []
        self.last_x: Optional[torch.Tensor] = None

    @staticmethod
    def _lam(sigma: float) -> float:
        sigma = min(max(sigma, 1e-6), 1 - 1e-6)
        return math.log((1 - sigma) / sigma)

    def _update(self, x, x0s, lams, s_cur, s_next, x0_new=None):
        """One UniPC update from sigma s_cur to s_next using stored x0 predictions (latest last).
        With x0_new (the prediction at s_next) it is the corrector, else the predictor."""
        a_next = 1 - s_next
        lam_c, lam_n = self._lam(s_cur), self._lam(s_next)
        h = lam_n - lam_c
        m0 = x0s[-1]
        hh = -h
        h_phi_1 = math.expm1(hh)
        B_h = math.expm1(hh)
        x_t = (s_next / max(s_cur, 1e-12)) * x - a_next * h_phi_1 * m0
        rks, D1s = [], []
        for k in range(1, len(x0s)):
            rk = (lams[-1 - k] - lam_c) / h
            rks.append(rk)
            D1s.append((x0s[-1 - k] - m0) / rk)
        if x0_new is None and not D1s:
            return x_t
        h_phi_k = h_phi_1 / hh - 1.0
        # order-2 closed forms (rhos = 0.5) as in the UniPC paper's bh variants
        if x0_new is None:
            return x_t - a_next * B_h * 0.5 * D1s[0]
        corr = 0.0
        if D1s:
            # solve the 2x2 system for (rho_p, rho_c)
            r = rks[0]
            b1 = h_phi_k / B_h
            h_phi_k2 = h_phi_k / hh - 0.5
            b2 = h_phi_k2 * 2.0 / B_h
            # R = [[1, 1], [r, 1]] ; b = [b1, b2]
            det = 1.0 - r
            rho_p = (b1 - b2) / det if abs(det) > 1e-12 else 0.0
            rho_c = b1 - rho_p
            corr = rho_p * D1s[0]
        else:
            rho_c = 0.5
        D1_t = x0_new - m0
        return x_t - a_next * B_h * (corr + rho_c * D1_t)

    # ------------------------------------------------------------------ the step as linear combinations
    def _coeffs(self, n_hist: int, lams: List[float], s_cur: float, s_next: float, corrector: bool):
        """Scalar weights of one `_update`: the result is cx * x + c0 * m0 + c1 * m_prev (+ cn * x0_new for the
        corrector), with m0 / m_prev the latest / second-latest stored predictions (`n_hist` of them exist)."""
        a_next = 1 - s_next
        lam_c, lam_n = self._lam(s_cur), self._lam(s_next)
        h = lam_n - lam_c
        hh = -h
        h_phi_1 = math.expm1(hh)
        B_h = math.expm1(hh)
        cx = s_next / max(s_cur, 1e-12)
        c0 = -a_next * h_phi_1
        c1 = cn = 0.0
        rk = (lams[-2] - lam_c) / h if n_hist > 1 else None
        if not corrector:
            if rk is not None:
                c1 = -a_next * B_h * 0.5 / rk
                c0 += a_next * B_h * 0.5 / rk
            return cx, c0, c1, cn
        h_phi_k = h_phi_1 / hh - 1.0
        if rk is not None:
            b1 = h_phi_k / B_h
            h_phi_k2 = h_phi_k / hh - 0.5
            b2 = h_phi_k2 * 2.0 / B_h
            det = 1.0 - rk
            rho_p = (b1 - b2) / det if abs(det) > 1e-12 else 0.0
            rho_c = b1 - rho_p
            c1 = -a_next * B_h * rho_p / rk
            c0 += a_next * B_h * rho_p / rk
        else:
            rho_c = 0.5
        cn = -a_next * B_h * rho_c
        c0 += a_next * B_h * rho_c
        return cx, c0, c1, cn

    def plan(self) -> dict:
        """Weights of the current step (index self.i), for the eager path and for the fused CFG + UniPC kernel:
            x0  = x - s_cur * v
            xf  = cL * L + cP * P + cP2 * P2 + cX0 * x0     (corrector; only when `correct`)   else xf = x
            x0  = xf - s_cur * v                                                     (again, after the corrector)
            out = dX * xf + dX0 * x0 + dP * P               (predictor)              or out = x0 when `final`
        with L the latent that entered the previous step (after its corrector), P / P2 the previous / second-previous
        stored predictions. Afterwards L <- xf, P2 <- P, P <- x0."""
        s_cur = float(self.sigmas[self.i])
        s_next = float(self.sigmas[self.i + 1])
        n = len(self.lam_hist)
        out = {"s_cur": s_cur, "correct": False, "final": s_next <= 0.0, "cL": 0.0, "cP": 0.0, "cP2": 0.0, "cX0": 0.0,
               "dX": 0.0, "dX0": 0.0, "dP": 0.0}
        if n >= 1 and s_cur > 0:
            s_prev = float(self.sigmas[self.i - 1])
            k = min(self.order, n)
            cx, c0, c1, cn = self._coeffs(k, self.lam_hist[-k:], s_prev, s_cur, corrector=True)
            out.update(correct=True, cL=cx, cP=c0, cP2=c1, cX0=cn)
        if not out["final"]:
            lams = (self.lam_hist + [self._lam(s_cur)])[-self.order:]
            cx, c0, c1, _ = self._coeffs(len(lams), lams, s_cur, s_next, corrector=False)
            out.update(dX=cx, dX0=c0, dP=c1)
        return out

    def device_state(self, like: torch.Tensor) -> dict:
        """Buffers of the fused kernel path: L (latent of the previous step), P / P2 (latest / second-latest stored
        predictions), n = how many predictions are stored. Allocated once per generation."""
        if getattr(self, "_dev", None) is None or self._dev["L"].shape != like.shape:
            self._dev = {"L": torch.zeros_like(like), "P": torch.zeros_like(like), "P2": torch.zeros_like(like), "n": 0}
        return self._dev

    def advance(self) -> None:
        """Book-keeping after a step whose tensors were updated elsewhere (the fused kernel)."""
        self.lam_hist.append(self._lam(float(self.sigmas[self.i])))
        self.i += 1

    def step(self, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        pl = self.plan()
        s_cur = pl["s_cur"]
        xf = x.float()
        vf = v.float()
        x0 = xf - s_cur * vf
        P = self.x0_hist[-1] if self.x0_hist else None
        P2 = self.x0_hist[-2] if len(self.x0_hist) > 1 else None
        if pl["correct"]:
            xf = pl["cL"] * self.last_x + pl["cP"] * P + pl["cX0"] * x0
            if P2 is not None and pl["cP2"] != 0.0:
                xf = xf + pl["cP2"] * P2
            x0 = xf - s_cur * vf
        self.x0_hist.append(x0)
        self.x0_hist = self.x0_hist[-2:]
        self.last_x = xf
        if pl["final"]:
            out = x0
        else:
            out = pl["dX"] * xf + pl["dX0"] * x0
            if P is not None and pl["dP"] != 0.0:
                out = out + pl["dP"] * P
        self.advance()
        return out.to(x.dtype)


def make_sampler(kind: str, sigmas: torch.Tensor):
    if kind == "euler":
        return EulerSampler(sigmas)
    if kind == "unipc":
        return UniPCSampler(sigmas)
    raise ValueError(f"unknown scheduler {kind!r}")
