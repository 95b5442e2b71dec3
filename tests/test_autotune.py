"""Autotuner selection logic (CPU, with an injected timer) and one run on the GPU."""

import json

import numpy as np
import pytest

from mytriton_b200 import kernels as corpus
import mytriton_b200 as triton
from mytriton_b200.autotune import Autotuner, Config

CONFIGS = [Config({"BLOCK": 256}, num_warps=2), Config({"BLOCK": 1024}, num_warps=4),
           Config({"BLOCK": 4096}, num_warps=8)]


class FakeDeviceArray:
    """Looks like a device array to the tuner; never launched (the timer is faked)."""

    def __init__(self, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (4096, False),
                                         "version": 3, "strides": None}


def grid_for(n):
    return lambda meta: (triton.cdiv(n, meta["BLOCK"]),)


def test_host_arguments_use_first_config_and_time_nothing():
    calls = []
    tuner = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"], timer=lambda *a: calls.append(a) or 1.0)
    x = np.zeros(1000, np.float32)
    _, _, src = tuner[grid_for(1000)](x, x, 1000)
    assert calls == []
    assert "__launch_bounds__(64)" in src          # num_warps=2 of the first config


def test_picks_fastest_and_caches_per_key(monkeypatch, tmp_path):
    timings = {"BLOCK=256, num_warps=2": 3.0, "BLOCK=1024, num_warps=4": 1.0, "BLOCK=4096, num_warps=8": 2.0}
    seen = []

    class FakeLauncher:
        def __init__(self, label):
            self.label = label

    def fake_launcher(grid, *args, **kwargs):
        label = ", ".join(f"{k}={kwargs[k]}" for k in ("BLOCK", "num_warps"))
        seen.append(label)
        return FakeLauncher(label)

    def fake_timer(run, stream_of, warmup, rep):
        return timings[run.label]

    monkeypatch.setattr(corpus.relu_kernel, "launcher", fake_launcher)
    cache_file = tmp_path / "tune.json"
    tuner = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"], timer=fake_timer, cache_path=cache_file)
    x = FakeDeviceArray(5000)
    best = tuner.best_config(grid_for(5000), (x, x, 5000), {})
    assert best.kwargs == {"BLOCK": 1024} and best.num_warps == 4
    assert len(seen) == 3
    tuner.best_config(grid_for(5000), (x, x, 5000), {})
    assert len(seen) == 3                                   # cached
    tuner.best_config(grid_for(7000), (FakeDeviceArray(7000),) * 2 + (7000,), {})
    assert len(seen) == 6                                   # new key -> tuned again
    stored = json.loads(cache_file.read_text())["relu_kernel"]
    assert {tuple(e["key"]) for e in stored} == {("5000", "x:float32", "out:float32"),
                                                  ("7000", "x:float32", "out:float32")}
    # a fresh tuner starts from the file
    again = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"], timer=fake_timer, cache_path=cache_file)
    assert again.best_config(grid_for(5000), (x, x, 5000), {}).num_warps == 4
    assert len(seen) == 6


def test_config_that_cannot_compile_is_skipped(monkeypatch):
    def fake_launcher(grid, *args, **kwargs):
        if kwargs["BLOCK"] == 256:
            raise ValueError("does not fit")
        return kwargs["BLOCK"]

    monkeypatch.setattr(corpus.relu_kernel, "launcher", fake_launcher)
    tuner = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"], timer=lambda run, *a: 1.0 / run)
    x = FakeDeviceArray(100)
    assert tuner.best_config(grid_for(100), (x, x, 100), {}).kwargs == {"BLOCK": 4096}


@pytest.mark.gpu
def test_autotuned_kernel_on_gpu(gpu):
    from mytriton_b200 import device, runtime

    n = 1 << 20
    rng = np.random.default_rng(0)
    x = rng.standard_normal(n, dtype=np.float32)
    dx, dout = device.to_device(x), device.empty(n)
    tuner = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"])
    tuner[grid_for(n)](dx, dout, n)
    runtime.synchronize()
    assert np.array_equal(dout.to_host(), np.maximum(x, np.float32(0)))
    (key, chosen), = tuner.cache.items()
    assert chosen in CONFIGS and all(np.isfinite(v) for v in tuner.timings[key].values())


@triton.jit
def bucket_total_kernel(x, total, n, BLOCK: triton.language.constexpr):
    offs = triton.language.program_id(0) * BLOCK + triton.language.arange(0, BLOCK)
    v = triton.language.load(x + offs, mask=offs < n, other=0.0)
    triton.language.atomic_add(total, triton.language.sum(v))


def test_accumulating_kernels_are_not_tuned_on_live_buffers_unless_told_how_to_reset():
    tuner = Autotuner(bucket_total_kernel, CONFIGS[:2], key=["n"], timer=lambda *a: 1.0)
    x, total = FakeDeviceArray(4096), FakeDeviceArray(1)
    with pytest.raises(ValueError, match="reset_to_zero"):
        tuner.best_config(grid_for(4096), (x, total, 4096), {})
    with pytest.raises(ValueError, match="no parameter of the kernel"):
        Autotuner(bucket_total_kernel, CONFIGS[:2], key=["n"], reset_to_zero=["sum"])


def test_stored_timings_from_another_platform_are_ignored(tmp_path, monkeypatch):
    cache_file = tmp_path / "tune.json"
    entry = {"key": ["5000", "x:float32", "out:float32"], "config": CONFIGS[2].label(), "ms": {}}
    cache_file.write_text(json.dumps({"relu_kernel": [dict(entry, platform="some other GPU / mtb200 0.0")]}))
    tuner = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"], cache_path=cache_file)
    assert tuner.cache == {}
    cache_file.write_text(json.dumps({"relu_kernel": [dict(entry, platform=tuner._platform())]}))
    tuner = Autotuner(corpus.relu_kernel, CONFIGS, key=["n"], cache_path=cache_file)
    assert list(tuner.cache.values()) == [CONFIGS[2]]
    # saving goes through a rename: no partial file, no stray temporary
    tuner._save_disk_cache()
    assert [p.name for p in tmp_path.iterdir()] == ["tune.json"]
    assert json.loads(cache_file.read_text())["relu_kernel"][0]["platform"] == tuner._platform()


@pytest.mark.gpu
def test_tuning_an_accumulating_kernel_leaves_one_launch_worth_of_result(gpu):
    from mytriton_b200 import device, runtime

    n = 1 << 16
    x = np.ones(n, dtype=np.float32)
    dx, total = device.to_device(x), device.to_device(np.zeros(1, np.float32))
    tuner = Autotuner(bucket_total_kernel, CONFIGS[:2], key=["n"], reset_to_zero=["total"])
    tuner[grid_for(n)](dx, total, n)                 # tunes (many trial launches), then launches once
    runtime.synchronize()
    assert total.to_host()[0] == float(n)
    keep = device.to_device(np.full(1, 5.0, np.float32))
    tuner = Autotuner(bucket_total_kernel, CONFIGS[:2], key=["n"], restore_value=["total"])
    tuner[grid_for(n)](dx, keep, n)
    runtime.synchronize()
    assert keep.to_host()[0] == 5.0 + float(n)
