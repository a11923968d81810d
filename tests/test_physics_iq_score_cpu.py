"""Built-in Physics-IQ scorer on synthetic clips whose motion is known."""
import json

import numpy as np
import pytest

from cosmos_b200.evaluation import physics_iq_score as ps


def _clip(path_x, path_y, n=12, size=48, box=8, start=0):
    """A bright square that moves along (path_x[t], path_y[t]) from frame `start` on; still before."""
    frames = np.full((n, size, size, 3), 20, dtype=np.uint8)
    for t in range(n):
        k = max(0, t - start)
        x, y = path_x[min(k, len(path_x) - 1)], path_y[min(k, len(path_y) - 1)]
        frames[t, y:y + box, x:x + box] = 230
    return frames


def test_measures_order_clips_by_how_well_the_motion_matches():
    xs = list(range(2, 38, 3))
    real = _clip(xs, [10] * 12)
    same = ps.compare(real, real)
    assert same["spatial_iou"] == same["spatiotemporal_iou"] == same["weighted_spatial_iou"] == 1.0 and same["mse"] == 0.0
    late = ps.compare(_clip(xs, [10] * 12, start=4), real)            # right place, wrong time
    assert late["spatial_iou"] > 0.6 and late["spatiotemporal_iou"] < 0.5 * late["spatial_iou"]
    elsewhere = ps.compare(_clip(xs, [34] * 12), real)                # right time, wrong place
    assert elsewhere["spatial_iou"] < 0.05 and elsewhere["weighted_spatial_iou"] < 0.05
    still = ps.compare(_clip([2], [10]), real)                        # nothing moves
    assert still["spatial_iou"] == 0.0 and 0.0 < still["mse"] < late["mse"] + 1.0
    scores = [ps.physics_iq(m) for m in (same, late, elsewhere)]
    assert scores[0] == 100.0 and scores[0] > scores[1] > scores[2] >= 0.0
    # two empty motion fields agree
    flat = np.full((5, 16, 16, 3), 7, dtype=np.uint8)
    assert ps.compare(flat, flat)["spatiotemporal_iou"] == 1.0
    with pytest.raises(ValueError):
        ps.compare(real, real[:, :40])
    with pytest.raises(ValueError):
        ps.compare(real[:1], real[:1])


def test_physical_variance_normalises_the_score():
    xs = list(range(2, 38, 3))
    real1, real2 = _clip(xs, [10] * 12), _clip(xs, [12] * 12)         # two takes of the scene differ a little
    var = ps.compare(real2, real1)
    gen = _clip(xs, [11] * 12)
    raw = ps.compare(gen, real1)
    assert ps.physics_iq(raw, var) == 100.0 > ps.physics_iq(raw)       # as close as a second real take: full marks
    far = ps.compare(_clip(xs, [30] * 12), real1)
    assert ps.physics_iq(far, var) < 40.0


def test_directory_scoring_writes_csv_and_summary(tmp_path, capsys):
    xs = list(range(2, 38, 3))
    gen_dir, real_dir, take2 = tmp_path / "staged", tmp_path / "real", tmp_path / "take2"
    for d in (gen_dir, real_dir, take2):
        d.mkdir()
    np.save(real_dir / "0001_ball.npy", _clip(xs, [10] * 12))
    np.save(take2 / "0001_ball.npy", _clip(xs, [12] * 12))
    np.save(gen_dir / "0001_ball.npy", _clip(xs, [11] * 12))
    np.save(real_dir / "0002_block.npy", _clip(xs, [20] * 12, size=64))          # another size: resized to the staged clip
    np.save(gen_dir / "0002_block.npy", _clip(xs, [30] * 12))
    np.save(gen_dir / "0003_no_truth.npy", _clip(xs, [30] * 12))                 # no real clip: skipped
    rc = ps.main(["--generated_videos_dir", str(gen_dir), "--results_dir", str(tmp_path / "res"), "--physics_iq_dir",
                  str(real_dir), "--real_take2_dir", str(take2), "--fps", "24", "--device", "cpu"])
    assert rc == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary["cases"] == 2 and summary == json.loads((tmp_path / "res" / "summary.json").read_text())
    rows = (tmp_path / "res" / "per_case.csv").read_text().splitlines()
    assert rows[0] == "case,spatial_iou,spatiotemporal_iou,weighted_spatial_iou,mse,physics_iq" and len(rows) == 3
    assert rows[1].startswith("0001_ball,") and float(rows[1].split(",")[-1]) > float(rows[2].split(",")[-1])
    with pytest.raises(ValueError):
        ps.score_directory(gen_dir, tmp_path / "res", tmp_path / "res2")
