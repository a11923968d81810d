"""Reasoner prompting conventions (utils/reasoner_prompts.py)."""
import pytest

from cosmos_b200.utils import reasoner_prompts as rp


def test_presets_and_message_layout():
    assert (rp.DECODING_DIRECT.temperature, rp.DECODING_DIRECT.top_p, rp.DECODING_DIRECT.presence_penalty) == (0.7, 0.8, 1.5)
    assert (rp.DECODING_REASONING.temperature, rp.DECODING_REASONING.top_p, rp.DECODING_REASONING.presence_penalty) == (0.6, 0.95, 0.0)
    assert rp.decoding_for(True, max_new_tokens=64).max_new_tokens == 64 and rp.DECODING_REASONING.max_new_tokens != 64
    m = rp.build_messages("What happens?", images=["file:///a.jpg"], videos=["file:///b.mp4"], reasoning=True)
    assert m[0] == {"role": "system", "content": "You are a helpful assistant."}
    kinds = [p["type"] for p in m[1]["content"]]
    assert kinds == ["image_url", "video_url", "text"]                  # media before text
    assert m[1]["content"][-1]["text"].startswith("What happens?") and "<think>" in m[1]["content"][-1]["text"]
    assert rp.build_messages("hi", system=None)[0]["role"] == "user"


def test_split_reasoning_variants():
    assert rp.split_reasoning("<think>\nstep 1\n</think>\n\nThe cup.") == ("step 1", "The cup.")
    assert rp.split_reasoning("The cup.") == ("", "The cup.")
    assert rp.split_reasoning("<think>cut off mid") == ("cut off mid", "")
    assert rp.split_reasoning("already open\n</think> done") == ("already open", "done")


def test_coordinates_round_trip_per_axis():
    assert rp.to_normalized([640, 360, 1280, 720], 1280, 720) == [500, 500, 1000, 1000]
    assert rp.to_normalized([-5, 800], 1280, 720) == [0, 1000]                 # clamped
    assert rp.from_normalized([214, 141, 497, 722], 1000, 2000) == [214.0, 282.0, 497.0, 1444.0]
    px = [100.0, 50.0]
    back = rp.from_normalized(rp.to_normalized(px, 640, 480), 640, 480)
    assert abs(back[0] - px[0]) < 0.7 and abs(back[1] - px[1]) < 0.5


def test_answer_parsers():
    ans = ('<think>the load is left of [the] door {maybe}</think>\nHere it is:\n```json\n[\n  {"bbox_2d": [214, 141, 497, 722], '
           '"label": "load as a whole"}\n]\n```')
    assert rp.parse_boxes(ans) == [{"bbox_2d": [214.0, 141.0, 497.0, 722.0], "label": "load as a whole"}]
    assert rp.parse_boxes(ans, 1000, 500)[0]["bbox_2d"] == [214.0, 70.5, 497.0, 361.0]
    traj = 'Sure: [{"point_2d": [721, 674], "label": "gripper trajectory"}, {"point_2d": [549, 745], "label": "gripper trajectory"}] done'
    pts = rp.parse_points(traj, 1000, 1000)
    assert [p["point_2d"] for p in pts] == [[721.0, 674.0], [549.0, 745.0]]
    assert rp.parse_points('{"point_2d": [1, 2], "label": "a"}')[0]["label"] == "a"      # a single object
    ev = rp.parse_events('[{"start": "00:01.50", "end": "01:02.25", "caption": "walks"}, {"start": 3, "end": 4.5, "caption": "sits"}]')
    assert ev == [{"start": 1.5, "end": 62.25, "caption": "walks"}, {"start": 3.0, "end": 4.5, "caption": "sits"}]
    assert rp.parse_boxes('[{"bbox_2d": [1, 2, 3], "label": "short"}, "noise"]') == []
    with pytest.raises(ValueError):
        rp.parse_json_answer("no structured content here")


def test_timestamps():
    assert rp.parse_timestamp("01:02.25") == 62.25 and rp.parse_timestamp("7s") == 7.0 and rp.parse_timestamp("1:00:01") == 3601.0
    assert rp.format_timestamp(62.25) == "01:02.25" and rp.format_timestamp(0) == "00:00.00"
    assert rp.parse_timestamp(rp.format_timestamp(125.37)) == pytest.approx(125.37)
    with pytest.raises(ValueError):
        rp.parse_timestamp("1:2:3:4")


def test_task_prompts_name_the_keys_the_parsers_read():
    assert "bbox_2d" in rp.grounding_prompt("the red cup") and "0-1000" in rp.grounding_prompt("x")
    assert "point_2d" in rp.trajectory_prompt("Move the bowl")
    assert "'start', 'end' and 'caption'" in rp.events_prompt() and "mm:ss.ff" in rp.events_prompt("mm:ss.ff")
    with pytest.raises(ValueError):
        rp.events_prompt("frames")
