"""The CPU restatement of tnsr's forty_five model against the reference's own fixture."""
import json
import os

import numpy as np
import pytest

from oracle import forty_five
from tnsr_b200.parameters import NamedParameters

FIXTURES = os.path.join(os.path.dirname(__file__), "golden", "forty_five")


def test_forward_matches_the_reference_fixture():
    """examples/forty_five/tests.rs:2-47: logits and values of `fixtures/tiny` within 2e-5 of reference.json."""
    named, config = NamedParameters.load(os.path.join(FIXTURES, "tiny"))
    reference = json.load(open(os.path.join(FIXTURES, "tiny", "reference.json")))
    model = forty_five.Model(named, config)
    batch = reference["batch"]
    logits, values = model.forward(batch["token_ids"], batch["token_type_ids"], batch["phase_ids"])
    assert logits.shape == (2, 46) and values.shape == (2,)
    assert np.max(np.abs(logits - np.asarray(reference["logits"], dtype=np.float32))) < 2e-5
    assert np.max(np.abs(values - np.asarray(reference["values"], dtype=np.float32))) < 2e-5


def test_separate_critic_archive_runs_and_masks_padding():
    named, config = NamedParameters.load(os.path.join(FIXTURES, "tiny-separate"))
    assert config["use_separate_critic"] is True
    model = forty_five.Model(named, config)
    ids = [[3, 4, 5, 0, 0, 0, 0, 0, 0, 0, 7, 8, 9, 10, 11, 0], [0] * 16]
    kinds = [[0, 1, 2, 0, 0, 0, 0, 0, 0, 0, 1, 2, 3, 4, 5, 0], [0] * 16]
    a = model.encode("token_encoder", ids, kinds)
    ids2 = [row[:] for row in ids]
    ids2[0][3] = 0                                  # still padding: nothing may change
    assert np.array_equal(a, model.encode("token_encoder", ids2, kinds))
    ids2[0][2] = 6                                  # a live key changed: every live row of that sample changes
    b = model.encode("token_encoder", ids2, kinds)
    assert not np.array_equal(a[0, 0], b[0, 0]) and np.array_equal(a[1], b[1])
    logits, values = model.forward(ids, kinds, [1, 4])
    assert np.all(np.isfinite(logits)) and np.all(np.isfinite(values))
