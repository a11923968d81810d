"""Structured prompt schema and negative-prompt metadata rules (io/prompt_schema.py)."""
import json
from pathlib import Path

import pytest

from cosmos_b200.io import prompt_schema as ps
from cosmos_b200.io.spec import spec_from_dict

REF = Path(__file__).resolve().parents[2] / "reference" / "cookbooks" / "cosmos3" / "generator"


def _prompt(**extra):
    subj = {f: "x" for f in ps.SUBJECT_FIELDS}
    subj.update(number_of_subjects=1, number_of_arms=2, number_of_legs=2)
    obj = {"subjects": [subj], "background_setting": "a lab", "lighting": {f: "soft" for f in ps.NESTED_FIELDS["lighting"]},
           "cinematography": {"camera_motion": "static"}, "actions": [{"time": "0-2s", "description": "moves"}],
           "segments": [], "transitions": [], "temporal_caption": "a robot moves"}
    obj.update(extra)
    return obj


def test_validate_accepts_the_schema_and_names_what_is_off():
    assert ps.validate_prompt(_prompt()) == []
    t2i = _prompt(subject_details={"fabric": "silk"}, quadrant_scan={"top_left": "a"}, comprehensive_t2i_caption="c",
                  resolution={"W": 1280, "H": 720}, aspect_ratio="16,9")
    t2i["subjects"][0]["number_of_fingers"] = 10
    assert ps.validate_prompt(t2i) == []
    assert ps.validate_prompt(_prompt(physical_realism="floating objects")) == []
    bad = ps.validate_prompt(_prompt(mood="happy", fps="24", lighting={"colour": "red"}, actions=[{"when": "now"}],
                                     resolution={"W": 0, "H": 720}))
    assert "unknown key 'mood'" in bad and "'fps' must be a number" in bad and "unknown key 'lighting.colour'" in bad
    assert "unknown key 'actions[0].when'" in bad and "'resolution' needs positive integers W and H" in bad
    assert ps.parse_prompt("a plain sentence") is None and ps.parse_prompt("{broken") is None


@pytest.mark.skipif(not REF.exists(), reason="reference assets not mounted")
def test_every_prompt_asset_of_the_reference_conforms():
    files = sorted(REF.glob("audiovisual/assets/prompts/*/*.json")) + sorted(REF.glob("audiovisual/assets/negative_prompts/*/*.json")) \
        + sorted(REF.glob("transfer/assets/*/prompt.json"))
    assert len(files) >= 10
    for f in files:
        obj = json.loads(f.read_text())
        assert ps.validate_prompt(obj) == [], f


def test_metadata_block_uses_the_reference_spelling():
    assert ps.make_metadata(1280, 720, 169, 24) == {"resolution": {"W": 1280, "H": 720}, "aspect_ratio": "16,9",
                                                   "duration": "7s", "fps": 24}
    assert ps.make_metadata(736, 544, 1, 24, "4,3") == {"resolution": {"W": 736, "H": 544}, "aspect_ratio": "4,3"}


def test_negative_prompt_metadata_modes():
    pos = ps.compact(_prompt(resolution={"W": 1280, "H": 720}, aspect_ratio="16,9", duration="7s", fps=24))
    neg = ps.compact({"temporal_caption": "blurry", "physical_realism": "bad", "fps": 10, "duration": "2s"})
    none = json.loads(ps.negative_prompt_for(neg, pos, "none", False))
    assert none == {"temporal_caption": "blurry", "physical_realism": "bad"}
    same = json.loads(ps.negative_prompt_for(neg, pos, "same", False))
    assert same["fps"] == 24 and same["duration"] == "7s" and same["resolution"] == {"W": 1280, "H": 720}
    kept = json.loads(ps.negative_prompt_for(neg, pos, "same", True))
    assert kept["fps"] == 10 and kept["duration"] == "2s" and kept["aspect_ratio"] == "16,9"   # own keys win, the rest is copied
    kept_none = json.loads(ps.negative_prompt_for(neg, pos, "none", True))
    assert kept_none["fps"] == 10 and "resolution" not in kept_none
    # plain-text positive prompt: the metadata comes from the request
    fb = ps.make_metadata(320, 192, 49, 24)
    assert json.loads(ps.negative_prompt_for(neg, "a robot", "same", False, fb))["resolution"] == {"W": 320, "H": 192}
    assert ps.negative_prompt_for("ugly, blurry", pos, "same", False) == "ugly, blurry"
    with pytest.raises(ValueError):
        ps.negative_prompt_for(neg, pos, "mirror", False)


def test_spec_applies_the_negative_metadata_rules(tmp_path):
    (tmp_path / "neg.json").write_text(json.dumps({"temporal_caption": "static, blurry", "fps": 5}))
    base = dict(model_mode="text2video", name="s", prompt="a robot arm", negative_prompt_file="neg.json", num_frames=49,
                resolution="256", fps=24)
    s = spec_from_dict({**base, "negative_metadata_mode": "same"}, spec_dir=str(tmp_path))
    got = json.loads(s.negative_prompt_text((320, 192)))
    assert got == {"temporal_caption": "static, blurry", "resolution": {"W": 320, "H": 192}, "aspect_ratio": "16,9",
                   "duration": "2s", "fps": 24}
    s = spec_from_dict({**base, "negative_metadata_mode": "none", "negative_prompt_keep_metadata": True}, spec_dir=str(tmp_path))
    assert json.loads(s.negative_prompt_text((320, 192))) == {"temporal_caption": "static, blurry", "fps": 5}
    s = spec_from_dict({**base}, spec_dir=str(tmp_path))
    assert json.loads(s.negative_prompt_text()) == {"temporal_caption": "static, blurry"}
