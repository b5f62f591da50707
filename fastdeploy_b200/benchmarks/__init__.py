"""Workloads behind ``bench.py --config NAME``: each module builds its model from synthetic, random-initialised
files, runs the device-timed loop and the end-to-end loop (pinned host inputs in, results out) and returns the
keys of the benchmark's JSON line. Shared timing, clock sampling and process set-up live in :mod:`.common`.

The reference's counterparts are its per-model drivers (benchmark/cpp/benchmark_ppyoloe.cc,
benchmark/python/benchmark_ernie_seq_cls.py, benchmark/python/benchmark_ppocr.py) around the
``BENCHMARK_MODEL`` macro (benchmark/cpp/macros.h:20-116).
"""
