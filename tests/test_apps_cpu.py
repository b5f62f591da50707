"""Example applications: streaming VAD state machine and the DPM-Solver++ sampler."""
import numpy as np
import torch


def test_vad_segments_follow_the_hysteresis_and_cleanup_rules():
    from fastdeploy_b200.apps.silero_vad import Vad
    sr, frame_ms = 16000, 64
    # a stand-in model: probability = mean absolute amplitude of the window, state counts the windows
    def model(window, srate, h, c):
        assert window.shape == (1, sr // 1000 * frame_ms) and int(srate[0]) == sr
        return float(np.abs(window).mean()), h + 1, c
    vad = Vad(infer_fn=model, sample_rate=sr, frame_ms=frame_ms, threshold=0.5, min_silence_duration_ms=100)
    w = vad.window
    loud, quiet = np.full(w, 0.9, np.float32), np.full(w, 0.05, np.float32)
    # 0.32 s silence, 1.92 s speech, a 0.256 s dip (a segment closes once the silence has lasted 100 ms; its end is the
    # moment the silence began), 2.56 s speech, silence. A 1-window blip of silence inside speech changes nothing.
    audio = np.concatenate([quiet] * 5 + [loud] * 15 + [quiet] + [loud] * 14 + [quiet] * 4 + [loud] * 40 + [quiet] * 10)
    probs = vad.predict(audio)
    assert len(probs) == 89 and float(vad.h.reshape(-1)[0]) == 89.0          # the state is carried between windows
    assert [round(s, 3) for s in vad.starts] == [0.32, 2.496]
    assert [round(e, 3) for e in vad.ends] == [2.304, 5.12]
    raw = vad.get_result(remove_threshold=0.0, expand_head_threshold=0.0, expand_tail_threshold=0.0, merge_threshold=0.0)
    assert [(round(r["start"], 3), round(r["end"], 3)) for r in raw] == [(0.32, 2.304), (2.496, 5.12)]
    merged = vad.get_result(remove_threshold=1.6, expand_head_threshold=0.32, expand_tail_threshold=0.0, merge_threshold=0.3)
    assert [(round(r["start"], 3), round(r["end"], 3)) for r in merged] == [(0.0, 5.12)]
    only_long = vad.get_result(remove_threshold=2.0, expand_head_threshold=0.0, merge_threshold=0.0)
    assert [(round(r["start"], 3), round(r["end"], 3)) for r in only_long] == [(2.496, 5.12)]
    vad.reset()
    assert vad.predict(np.zeros(3 * w, np.float32)) == [0.0, 0.0, 0.0] and vad.get_result() == []


def test_dpm_solver_recovers_the_clean_sample_of_an_exact_noise_predictor():
    from fastdeploy_b200.apps.diffusion_schedulers import DPMSolverMultistepScheduler
    torch.manual_seed(0)
    x0 = torch.randn(2, 4, 8, 8, dtype=torch.float64)
    for order, solver in ((1, "midpoint"), (2, "midpoint"), (2, "heun"), (3, "midpoint")):
        sch = DPMSolverMultistepScheduler(beta_start=0.00085, beta_end=0.012, beta_schedule="scaled_linear",
                                          solver_order=order, solver_type=solver)
        sch.set_timesteps(20)
        assert list(sch.timesteps[:3]) == [999, 949, 899] and sch.timesteps[-1] == 50
        noise = torch.randn_like(x0)
        x = sch.add_noise(x0, noise, [999] * 2)
        for t in sch.timesteps:
            # an oracle that knows x0: eps = (x - alpha x0) / sigma; with it every order is exact
            eps = (x - float(sch.alpha_t[t]) * x0) / float(sch.sigma_t[t])
            x = sch.step(eps, int(t), sch.scale_model_input(x, t))
        a0, s0 = float(sch.alpha_t[0]), float(sch.sigma_t[0])
        # with an exact predictor every step keeps x = alpha x0 + sigma noise, for every order
        assert torch.allclose(x, a0 * x0 + s0 * noise, atol=1e-9)


def test_dpm_solver_first_step_matches_the_closed_form():
    from fastdeploy_b200.apps.diffusion_schedulers import DPMSolverMultistepScheduler
    sch = DPMSolverMultistepScheduler(solver_order=2)
    sch.set_timesteps(10)
    t, prev = int(sch.timesteps[0]), int(sch.timesteps[1])
    x = torch.full((1, 3), 2.0, dtype=torch.float64)
    eps = torch.full((1, 3), 0.5, dtype=torch.float64)
    out = sch.step(eps, t, x)
    a_s, s_s, a_t, s_t = sch.alpha_t[t], sch.sigma_t[t], sch.alpha_t[prev], sch.sigma_t[prev]
    x0 = (2.0 - s_s * 0.5) / a_s
    h = sch.lambda_t[prev] - sch.lambda_t[t]
    expect = s_t / s_s * 2.0 - a_t * (np.exp(-h) - 1.0) * x0
    assert torch.allclose(out, torch.full((1, 3), float(expect), dtype=torch.float64), atol=1e-12)
    betas = DPMSolverMultistepScheduler.betas_for_alpha_bar(50)
    assert betas.shape == (50,) and 0 < betas[0] < betas[-1] <= 0.999
