"""The measuring instruments that need the device: the kernel timeline of a decode step and the MMA issue-rate probe."""
import pytest
import torch

import tiny

pytestmark = pytest.mark.gpu


def test_decode_timeline_lists_the_steps_kernels_in_order(tmp_path):
    """One decode step of a tiny model: the embedding first, the sampler at the end, every layer's attention in between,
    every kernel ending after it starts and no earlier than the kernel before it ends."""
    from flambeau_b200.engine.step import Engine, EngineOptions
    from flambeau_b200.measure import workloads
    folder = tiny.make_folder(tmp_path / "m", tiny.CONFIG_A, seed=5, dtype="bfloat16")
    engine = Engine.from_folder(folder, EngineOptions(dtype="bfloat16", cache_tokens=512, max_requests=2,
                                                      max_step_tokens=8, max_seq_len=256))
    workloads.randomise_cache(engine)
    try:
        rows = workloads.decode_timeline(engine, 2, 100, torch.Generator().manual_seed(0))
    except workloads.TimelineUnavailable as exc:         # an instrument, not the engine: its absence fails nothing
        pytest.skip(f"no activity records here: {exc}")
    names = [n for _, _, n in rows]
    assert "embedding" in names[0] and any("sample" in n for n in names[-2:])
    layers = tiny.CONFIG_A["num_hidden_layers"]
    assert sum("attention" in n for n in names) == layers
    assert sum("rope_kv_write" in n for n in names) == layers
    last_end = 0.0
    for start, end, name in rows:
        assert end >= start >= 0.0, name
        assert end >= last_end - 1e-3, f"{name} ends before the kernel ahead of it"
        last_end = end
    engine.runtime.check_status("timeline")


def test_mma_issue_rate_probe_runs_and_reports_sane_cycles():
    """The probe compiles into the build folder, runs, and reports between 30 and 400 cycles per instruction for
    every stream; an MMA of 256 columns costs more than one of 128."""
    from flambeau_b200.measure.probes import run_probe
    table = run_probe("mma_issue_rate")
    rows = [ln.rsplit(None, 4) for ln in table.splitlines()[1:] if ln.strip()]
    assert len(rows) == 9
    each = {r[0].strip(): float(r[3]) for r in rows}
    assert all(30.0 < v < 400.0 for v in each.values()), each
    assert each["S-shaped, N = 256"] > 1.3 * each["S-shaped, N = 128"]
