"""Tile tuner: the search logic and the on-disk cache on a CPU (fake clock), and one real search on a GPU."""
import json

import pytest
import torch

from viola_b200 import tuning


@pytest.fixture()
def private_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("VIOLA_B200_CACHE", str(tmp_path))
    tuning.forget()
    yield tmp_path
    tuning.forget()
    tuning.enable(False)


def fake_search(signature, cost, *, unstable=()):
    state = {"tile": None, "calls": 0}
    buffer = torch.zeros(4)

    def run(tile):
        state["tile"] = tile
        state["calls"] += 1
        buffer.fill_(float(state["calls"]) if tile in unstable else 1.0)

    return tuning.search(signature, run, lambda: buffer, measure=lambda fn: (fn(), cost[state["tile"]])[1])


def test_search_picks_the_fastest_beyond_the_margin_and_persists(private_cache):
    signature = (0, (4096, 1152), (3456, 1152), "e4m3", "e4m3", "bf16", False, False, 1, True, 0, False)
    assert fake_search(signature, {0: 1.00, 128: 1.00, 256: 0.80}) == 256
    files = list((private_cache / "linear").glob("*.json"))
    assert len(files) == 1
    record = json.loads(files[0].read_text())
    assert record["tile"] == 256 and set(record["milliseconds"]) == {"0", "128", "256"}
    tuning.forget()                                            # a new process: the file answers, nothing is timed
    assert tuning.recall(signature) == 256
    assert tuning.choose(signature, None, None) == 256


def test_heuristic_stays_within_the_margin_and_unstable_candidates_are_rejected(private_cache):
    a = (1, (1152, 1152), (1152, 1152), "bf16", "bf16", "bf16", False, False, 14, False, 0, False)
    assert fake_search(a, {0: 1.00, 128: 0.99, 256: 1.20}) == 0           # 1 % is inside the 3 % margin
    b = (1, (1152, 3456), (1152, 3456), "bf16", "bf16", "bf16", False, False, 14, False, 0, False)
    assert fake_search(b, {0: 1.00, 128: 1.10, 256: 0.50}, unstable={256}) == 0
    assert tuning.log[-1][1].keys() == {0, 128}                           # the unstable one was never timed
    assert (private_cache / "orthogonalize").is_dir()


def test_without_tuning_nothing_is_searched(private_cache):
    tuning.enable(False)
    signature = (0, (128, 256), (512, 256), "e4m3", "e4m3", "bf16", False, False, 1, False, 0, False)
    assert tuning.choose(signature, lambda tile: pytest.fail("must not run"), None) == 0
    assert not list(private_cache.glob("*/*.json"))


@pytest.mark.gpu
def test_first_use_search_on_the_gpu_records_a_choice_and_keeps_results(private_cache):
    from viola_b200 import ops
    from viola_b200.nn import Linear
    torch.manual_seed(0)
    layer = Linear(1152, 3456, device="cuda", dtype=torch.bfloat16, autotune=True)        # switches tuning on
    x = torch.randn(2048, 1152, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    y.float().square().mean().backward()
    searched = [entry for entry in tuning.log if entry[0][0] == 0]
    assert searched and all(set(times) >= {0, 128, 256} for _, times, _ in searched)
    assert list(private_cache.glob("linear/*.json"))
    tuning.enable(False)
    tuning.forget()
    again = Linear(1152, 3456, device="cuda", dtype=torch.bfloat16)
    again.load_state_dict(layer.state_dict())
    assert torch.equal(again(x.detach()), y.detach())                     # the tile width never changes the result
    ops.check_status()
