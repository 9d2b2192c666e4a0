"""A step that fails on the host leaves the engine as it found it: the requests it brought in are gone again, no
page is lost, and the next step runs."""
import pytest
import torch

import tiny

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def engine(tmp_path_factory):
    from flambeau_b200.engine.step import Engine, EngineOptions
    folder = tiny.make_folder(tmp_path_factory.mktemp("fail"), tiny.CONFIG_A, seed=1, dtype="float32")
    return Engine.from_folder(folder, EngineOptions(dtype="float32", cache_tokens=64, max_requests=3,
                                                    max_step_tokens=32, max_seq_len=64))


def settled(engine, live=()):
    engine.cache.check_invariants()
    assert sorted(engine.cache.requests) == sorted(live)
    held = sum(1 for r in engine.cache.requests.values() for p in r.pages[0] if p >= 0)
    assert held + engine.cache.free_pages()[0] == engine.cache.groups[0].pool.n_pages


def test_failures_before_anything_runs(engine):
    from flambeau_b200.cache.pages import OutOfPages
    from flambeau_b200.engine.batch import BatchError, Entry
    engine.cache.release_all()
    engine.step([Entry("keep", [1, 2, 3], [2])])                       # a live request that must survive it all
    feed = torch.zeros(4, dtype=torch.int32, device="cuda")
    cases = [
        (BatchError, dict(entries=[Entry("a", [1, 2], [0])], token_feed=feed)),         # a feed needs single tokens
        (BatchError, dict(entries=[Entry("a", [1], [0]), Entry("b", [2], [0])], token_feed=feed[:1])),
        (BatchError, dict(entries=[Entry("a", [9999], [0])])),                            # token outside the vocabulary
        (BatchError, dict(entries=[Entry("a", [1, 2], [5])])),                            # wanted place outside the entry
        (BatchError, dict(entries=[Entry("a", [1]), Entry("a", [2])])),                   # a request twice
        (OutOfPages, dict(entries=[Entry("a", list(range(30))), Entry("b", list(range(30)))])),
        (BatchError, dict(entries=[Entry("a", list(range(40)))])),                        # more rows than a step may bring
    ]
    for error, kw in cases:
        with pytest.raises(error):
            engine.step(kw["entries"], token_feed=kw.get("token_feed"))
        settled(engine, live=["keep"])
    assert engine.cache.length("keep") == 3
    logits = engine.step([Entry("keep", [4], [0]), Entry("a", [5, 6], [1])], end=["a"])
    assert logits.shape[0] == 2 and torch.isfinite(logits).all()
    settled(engine, live=["keep"])
    engine.cache.release_all()


def test_a_launch_that_is_refused(engine, monkeypatch):
    """Nothing ran: the request the step brought in leaves again, and a live request has not grown."""
    from flambeau_b200.engine.batch import Entry
    from flambeau_b200.kernels.library import KernelError
    engine.cache.release_all()
    engine.step([Entry("keep", [1, 2, 3], [])])

    def refuse(batch):
        raise KernelError("gemm_tc: refused for the test")
    monkeypatch.setattr(engine, "_run", refuse)
    with pytest.raises(KernelError):
        engine.step([Entry("keep", [4], [0]), Entry("new", [7, 8], [1])])
    monkeypatch.undo()
    settled(engine, live=["keep"])
    assert engine.cache.length("keep") == 3
    logits = engine.step([Entry("keep", [4], [0]), Entry("new", [7, 8], [1])], end=["keep", "new"])
    assert torch.isfinite(logits).all()
    settled(engine)
