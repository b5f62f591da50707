"""Streaming voice-activity detection with a Silero-VAD style recurrent model.

The network takes a window of samples plus its LSTM state (``input [1, W]``, ``sr``, ``h``, ``c``) and returns the
speech probability of the window and the next state. The class feeds consecutive windows, keeps the state between
calls, runs the start / end hysteresis (a segment opens at ``threshold``, closes after ``min_silence`` below
``threshold - 0.15``) and cleans the segment list (drop short ones, pad head and tail, merge close neighbours).

Counterpart: examples/audio/silero-vad/cpp/vad.cc:25-257."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np


class Vad:
    def __init__(self, model_file: str = "", runtime_option=None, *, sample_rate: int = 16000, frame_ms: int = 64,
                 threshold: float = 0.5, min_silence_duration_ms: int = 0, speech_pad_ms: int = 0,
                 infer_fn: Optional[Callable] = None):
        """``infer_fn(window [1, W] fp32, sr int64 [1], h, c) -> (prob, h, c)`` replaces the runtime (tests, other
        models); otherwise ``model_file`` is loaded through :class:`fastdeploy_b200.Runtime`."""
        self.sample_rate, self.frame_ms, self.threshold = sample_rate, frame_ms, threshold
        self.sr_per_ms = sample_rate // 1000
        self.min_silence_samples = self.sr_per_ms * min_silence_duration_ms
        self.speech_pad_samples = self.sr_per_ms * speech_pad_ms
        self.window = frame_ms * self.sr_per_ms
        self._infer = infer_fn
        if infer_fn is None:
            import fastdeploy_b200 as fd
            opt = runtime_option or fd.RuntimeOption()
            opt.set_model_path(model_file, "", fd.ModelFormat.ONNX)
            self.runtime = fd.Runtime(opt)
            names = [self.runtime.get_input_info(i).name for i in range(self.runtime.num_inputs())]

            def run(window, sr, h, c):
                outs = self.runtime.infer(dict(zip(names, [window, sr, h, c])))
                return float(np.asarray(outs[0]).reshape(-1)[0]), np.asarray(outs[1]), np.asarray(outs[2])
            self._infer = run
        self.reset()

    def reset(self) -> None:
        self.h = np.zeros((2, 1, 64), np.float32)
        self.c = np.zeros((2, 1, 64), np.float32)
        self.triggered, self.temp_end, self.current_sample = False, 0, 0
        self.starts: List[float] = []
        self.ends: List[float] = []
        self.num_samples = 0

    # ------------------------------------------------------------------ streaming
    def accept_window(self, samples: np.ndarray) -> float:
        """One window of ``self.window`` samples in [-1, 1]; returns its speech probability."""
        w = np.asarray(samples, np.float32).reshape(1, -1)
        prob, self.h, self.c = self._infer(w, np.array([self.sample_rate], np.int64), self.h, self.c)
        self.current_sample += w.shape[1]
        self.num_samples += w.shape[1]
        if prob >= self.threshold and self.temp_end:
            self.temp_end = 0
        if prob >= self.threshold and not self.triggered:
            self.triggered = True
            start = self.current_sample - w.shape[1] - self.speech_pad_samples
            self.starts.append(start / self.sample_rate)
        if prob < self.threshold - 0.15 and self.triggered:
            if self.temp_end == 0:
                self.temp_end = self.current_sample
            if self.current_sample - self.temp_end >= self.min_silence_samples:
                end = self.temp_end + self.speech_pad_samples
                self.temp_end = 0
                self.triggered = False
                self.ends.append(end / self.sample_rate)
        return prob

    def predict(self, audio: Sequence[float]) -> List[float]:
        """A whole recording (the tail shorter than one window is zero padded); returns the per-window probabilities."""
        a = np.asarray(audio, np.float32).reshape(-1)
        n = (len(a) + self.window - 1) // self.window
        padded = np.zeros(n * self.window, np.float32)
        padded[:len(a)] = a
        probs = [self.accept_window(padded[i * self.window:(i + 1) * self.window]) for i in range(n)]
        self.num_samples = len(a)
        return probs

    # ------------------------------------------------------------------ segments
    def get_result(self, remove_threshold: float = 1.6, expand_head_threshold: float = 0.32,
                   expand_tail_threshold: float = 0.0, merge_threshold: float = 0.3) -> List[Dict[str, float]]:
        """Speech segments in seconds: segments shorter than ``remove_threshold`` go, every segment grows by the head
        / tail paddings without running into its neighbours, and segments closer than ``merge_threshold`` merge."""
        length = self.num_samples / self.sample_rate
        starts, ends = list(self.starts), list(self.ends)
        if not starts and not ends:
            return []
        if len(ends) != len(starts):
            ends.append(length)
        if remove_threshold < length:
            keep = [(s, e) for s, e in zip(starts, ends) if e - s >= remove_threshold]
            starts, ends = [s for s, _ in keep], [e for _, e in keep]
        if not starts:
            return []
        n = len(starts)
        new_s, new_e = list(starts), list(ends)
        for i in range(n):
            prev_end = ends[i - 1] if i > 0 else 0.0
            next_start = starts[i + 1] if i + 1 < n else length
            new_s[i] = max(starts[i] - expand_head_threshold, prev_end)
            new_e[i] = min(ends[i] + expand_tail_threshold, next_start)
        merged_s, merged_e = [new_s[0]], [new_e[0]]
        for s, e in zip(new_s[1:], new_e[1:]):
            if s - merged_e[-1] < merge_threshold:
                merged_e[-1] = e
            else:
                merged_s.append(s)
                merged_e.append(e)
        return [{"start": float(s), "end": float(e)} for s, e in zip(merged_s, merged_e)]
