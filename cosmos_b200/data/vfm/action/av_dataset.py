"""Constants of the autonomous-vehicle (AV) action domain (reference
cookbooks/cosmos3/generator/action/run_id_with_cosmos_framework.ipynb:661-670 quoting
cosmos_framework/data/vfm/action/av_dataset.py; action/README.md:29-41)."""
AV_ROTATION_FORMAT = "rot6d"
AV_POSE_CONVENTION = "backward_framewise"
AV_TRANSLATION_SCALE = 1.35
AV_ACTION_DIM = 9
AV_ACTION_CHUNK = 60
AV_FPS = 10
AV_PROMPT = "You are an autonomous vehicle planning system."

# raw action dimensionality per domain (README.md:107; action/README.md:29-35)
DOMAIN_ACTION_DIM = {
    "av": 9,
    "camera_pose": 9,
    "droid_lerobot": 10,
    "umi": 10,
    "bridge_orig_lerobot": 10,
    "egocentric": 57,
    "dual_arm": 20,
    "humanoid": 29,
}
DOMAIN_DEFAULTS = {
    "av": dict(action_chunk_size=60, fps=10, image_size=480),
    "droid_lerobot": dict(action_chunk_size=16, fps=15, image_size=480),
    "umi": dict(action_chunk_size=16, fps=20, image_size=256),
    "bridge_orig_lerobot": dict(action_chunk_size=16, fps=5, image_size=256),
    "camera_pose": dict(action_chunk_size=60, fps=10, image_size=480),
}
