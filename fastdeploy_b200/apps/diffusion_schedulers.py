"""Samplers of a latent-diffusion pipeline: DPM-Solver++ multistep (orders 1 - 3) on the variance-preserving noise
schedule, with the helpers a text-to-image loop needs (``set_timesteps``, ``scale_model_input``, ``step``,
``add_noise``). Tensors are torch tensors on any device; all arithmetic runs where the latents live.

With alpha_t = sqrt(prod(1 - beta)), sigma_t = sqrt(1 - alpha_t^2) and lambda_t = log(alpha_t / sigma_t), the
data-prediction form advances a sample from s to t by

    x_t = (sigma_t / sigma_s) x_s - alpha_t (exp(-h) - 1) D,        h = lambda_t - lambda_s,

where D is the predicted clean sample (order 1) or its multistep extrapolation (orders 2, 3).

Counterpart: examples/multimodal/stable_diffusion/cpp/dpm_solver_multistep_scheduler.cc:25-398."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch


class DPMSolverMultistepScheduler:
    def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.0001, beta_end: float = 0.02,
                 beta_schedule: str = "linear", trained_betas: Optional[Sequence[float]] = None, solver_order: int = 2,
                 predict_epsilon: bool = True, thresholding: bool = False, dynamic_thresholding_ratio: float = 0.995,
                 sample_max_value: float = 1.0, algorithm_type: str = "dpmsolver++", solver_type: str = "midpoint",
                 lower_order_final: bool = True):
        if trained_betas is not None and len(trained_betas):
            betas = np.asarray(trained_betas, np.float64)
        elif beta_schedule == "linear":
            betas = np.linspace(beta_start, beta_end, num_train_timesteps, dtype=np.float64)
        elif beta_schedule == "scaled_linear":
            betas = np.linspace(beta_start ** 0.5, beta_end ** 0.5, num_train_timesteps, dtype=np.float64) ** 2
        elif beta_schedule == "squaredcos_cap_v2":
            betas = self.betas_for_alpha_bar(num_train_timesteps)
        else:
            raise ValueError(f"unknown beta_schedule {beta_schedule!r}")
        if algorithm_type not in ("dpmsolver", "dpmsolver++") or solver_type not in ("midpoint", "heun"):
            raise ValueError("algorithm_type must be dpmsolver / dpmsolver++ and solver_type midpoint / heun")
        self.num_train_timesteps = num_train_timesteps
        self.betas = betas
        self.alphas_cumprod = np.cumprod(1.0 - betas)
        self.alpha_t = np.sqrt(self.alphas_cumprod)
        self.sigma_t = np.sqrt(1.0 - self.alphas_cumprod)
        self.lambda_t = np.log(self.alpha_t) - np.log(self.sigma_t)
        self.solver_order, self.predict_epsilon, self.thresholding = solver_order, predict_epsilon, thresholding
        self.dynamic_thresholding_ratio, self.sample_max_value = dynamic_thresholding_ratio, sample_max_value
        self.algorithm_type, self.solver_type, self.lower_order_final = algorithm_type, solver_type, lower_order_final
        self.init_noise_sigma = 1.0
        self.timesteps = np.arange(num_train_timesteps - 1, -1, -1, dtype=np.int64)
        self.num_inference_steps = None
        self.model_outputs: List[Optional[torch.Tensor]] = [None] * solver_order
        self.lower_order_nums = 0

    @staticmethod
    def betas_for_alpha_bar(n: int, max_beta: float = 0.999) -> np.ndarray:
        bar = lambda t: np.cos((t + 0.008) / 1.008 * np.pi / 2) ** 2
        return np.asarray([min(1 - bar((i + 1) / n) / bar(i / n), max_beta) for i in range(n)], np.float64)

    # ------------------------------------------------------------------ loop helpers
    def set_timesteps(self, num_inference_steps: int) -> None:
        self.num_inference_steps = num_inference_steps
        ts = np.linspace(0, self.num_train_timesteps - 1, num_inference_steps + 1).round()[::-1][:-1]
        self.timesteps = ts.astype(np.int64)
        self.model_outputs = [None] * self.solver_order
        self.lower_order_nums = 0

    def scale_model_input(self, sample: torch.Tensor, timestep=None) -> torch.Tensor:
        return sample

    def add_noise(self, original: torch.Tensor, noise: torch.Tensor, timesteps) -> torch.Tensor:
        t = np.asarray(timesteps, np.int64).reshape(-1)
        a = torch.as_tensor(self.alpha_t[t], dtype=original.dtype, device=original.device)
        s = torch.as_tensor(self.sigma_t[t], dtype=original.dtype, device=original.device)
        shape = [-1] + [1] * (original.dim() - 1)
        return a.view(shape) * original + s.view(shape) * noise

    # ------------------------------------------------------------------ solver
    def convert_model_output(self, model_output: torch.Tensor, timestep: int, sample: torch.Tensor) -> torch.Tensor:
        a, s = float(self.alpha_t[timestep]), float(self.sigma_t[timestep])
        if self.algorithm_type == "dpmsolver++":
            x0 = (sample - s * model_output) / a if self.predict_epsilon else model_output
            if self.thresholding:
                flat = x0.abs().reshape(x0.shape[0], -1).float()
                q = torch.quantile(flat, self.dynamic_thresholding_ratio, dim=1)
                q = torch.clamp(q, min=self.sample_max_value).view([-1] + [1] * (x0.dim() - 1)).to(x0.dtype)
                x0 = torch.maximum(torch.minimum(x0, q), -q) / q
            return x0
        return model_output if self.predict_epsilon else (sample - a * model_output) / s

    def _first_order(self, d, t, prev_t, sample):
        lam_t, lam_s = self.lambda_t[prev_t], self.lambda_t[t]
        a_t, s_t, s_s, a_s = self.alpha_t[prev_t], self.sigma_t[prev_t], self.sigma_t[t], self.alpha_t[t]
        h = lam_t - lam_s
        if self.algorithm_type == "dpmsolver++":
            return float(s_t / s_s) * sample - float(a_t * (np.exp(-h) - 1.0)) * d
        return float(a_t / a_s) * sample - float(s_t * (np.exp(h) - 1.0)) * d

    def _second_order(self, outs, ts, prev_t, sample):
        t, s0, s1 = prev_t, ts[-1], ts[-2]
        m0, m1 = outs[-1], outs[-2]
        lam_t, lam_s0, lam_s1 = self.lambda_t[t], self.lambda_t[s0], self.lambda_t[s1]
        h, h0 = lam_t - lam_s0, lam_s0 - lam_s1
        r0 = h0 / h
        d0, d1 = m0, (1.0 / r0) * (m0 - m1)
        a_t, s_t, s_s0, a_s0 = self.alpha_t[t], self.sigma_t[t], self.sigma_t[s0], self.alpha_t[s0]
        if self.algorithm_type == "dpmsolver++":
            e = np.exp(-h) - 1.0
            if self.solver_type == "midpoint":
                return float(s_t / s_s0) * sample - float(a_t * e) * d0 - float(0.5 * a_t * e) * d1
            return float(s_t / s_s0) * sample - float(a_t * e) * d0 + float(a_t * (e / h + 1.0)) * d1
        e = np.exp(h) - 1.0
        if self.solver_type == "midpoint":
            return float(a_t / a_s0) * sample - float(s_t * e) * d0 - float(0.5 * s_t * e) * d1
        return float(a_t / a_s0) * sample - float(s_t * e) * d0 - float(s_t * (e / h - 1.0)) * d1

    def _third_order(self, outs, ts, prev_t, sample):
        t, s0, s1, s2 = prev_t, ts[-1], ts[-2], ts[-3]
        m0, m1, m2 = outs[-1], outs[-2], outs[-3]
        lam = self.lambda_t
        h, h0, h1 = lam[t] - lam[s0], lam[s0] - lam[s1], lam[s1] - lam[s2]
        r0, r1 = h0 / h, h1 / h
        d0 = m0
        d1_0, d1_1 = (1.0 / r0) * (m0 - m1), (1.0 / r1) * (m1 - m2)
        d1 = d1_0 + float(r0 / (r0 + r1)) * (d1_0 - d1_1)
        d2 = float(1.0 / (r0 + r1)) * (d1_0 - d1_1)
        a_t, s_t, s_s0, a_s0 = self.alpha_t[t], self.sigma_t[t], self.sigma_t[s0], self.alpha_t[s0]
        if self.algorithm_type == "dpmsolver++":
            e = np.exp(-h) - 1.0
            return (float(s_t / s_s0) * sample - float(a_t * e) * d0 + float(a_t * (e / h + 1.0)) * d1
                    - float(a_t * ((e + h) / h ** 2 - 0.5)) * d2)
        e = np.exp(h) - 1.0
        return (float(a_t / a_s0) * sample - float(s_t * e) * d0 - float(s_t * (e / h - 1.0)) * d1
                - float(s_t * ((e - h) / h ** 2 - 0.5)) * d2)

    def step(self, model_output: torch.Tensor, timestep: int, sample: torch.Tensor) -> torch.Tensor:
        """One reverse step from ``timestep`` to the next entry of ``timesteps`` (0 after the last)."""
        if self.num_inference_steps is None:
            raise RuntimeError("call set_timesteps before step")
        idx = int(np.nonzero(self.timesteps == int(timestep))[0][0]) if int(timestep) in self.timesteps else len(self.timesteps) - 1
        prev_t = 0 if idx == len(self.timesteps) - 1 else int(self.timesteps[idx + 1])
        final = idx == len(self.timesteps) - 1 and self.lower_order_final and len(self.timesteps) < 15
        second_last = idx == len(self.timesteps) - 2 and self.lower_order_final and len(self.timesteps) < 15
        d = self.convert_model_output(model_output, int(timestep), sample)
        self.model_outputs = self.model_outputs[1:] + [d]
        if self.solver_order == 1 or self.lower_order_nums < 1 or final:
            prev = self._first_order(d, int(timestep), prev_t, sample)
        elif self.solver_order == 2 or self.lower_order_nums < 2 or second_last:
            ts = [int(self.timesteps[idx - 1]), int(timestep)]
            prev = self._second_order(self.model_outputs, ts, prev_t, sample)
        else:
            ts = [int(self.timesteps[idx - 2]), int(self.timesteps[idx - 1]), int(timestep)]
            prev = self._third_order(self.model_outputs, ts, prev_t, sample)
        if self.lower_order_nums < self.solver_order:
            self.lower_order_nums += 1
        return prev
