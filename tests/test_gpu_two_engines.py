"""Two engines in one process on two devices ("N GPUs are N engines"): the kernels' shared-memory opt-in is per device,
so the second engine's first step must work as the first's does. Skipped on a box with one GPU."""
import numpy as np
import pytest

import splosh_b200 as S
from helpers import tokens_for
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_a_second_engine_on_another_device_gives_the_same_logits():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU visible")
    g = S.tiny_geometry()
    model = O.Model(O.tiny_geometry())
    toks = tokens_for(0xD00D, 32, g.vocab)
    rows = [S.EngineRow(0, toks[p], p, p >= 20) for p in range(24)]
    logits = []
    for device in (0, 1):
        engine = S.Engine(g, S.EngineConfig(max_slots=2, max_rows=32, kv_pages=4, max_context=512, device=device))
        engine.load_model(model)
        engine.step(rows)
        logits.append(engine.all_logits())
    assert not np.isnan(logits[0]).any()
    assert np.array_equal(logits[0], logits[1])
