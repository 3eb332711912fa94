"""Checkpoint transforms for rendering (reference: landmark/render/util/utils.py:6-19)."""
import torch


def transform_gridnerf_model_to_channel_last(ckpt_path: str, out_path: str = None) -> str:
    """Write a copy of a GridNeRF checkpoint whose planes are stored ``[1, B, H, W, C]`` (channels last);
    the file gets the ``_channel_last.th`` suffix the reference uses.  Loading accepts both layouts."""
    state = torch.load(ckpt_path, map_location="cpu", weights_only=False)
    inner = state["state_dict"] if "state_dict" in state else state
    for key in list(inner.keys()):
        if "plane_coef" in key and inner[key].dim() == 5:
            inner[key] = inner[key].permute(0, 2, 3, 4, 1).contiguous()
    out_path = out_path or ckpt_path.replace(".th", "_channel_last.th")
    torch.save(state, out_path)
    return out_path


_GS_MLP_KEYS = {"opacity_mlp": "anchor_decoder.mlp_opacity", "cov_mlp": "anchor_decoder.mlp_cov",
                "color_mlp": "anchor_decoder.mlp_color", "mlp_feature_bank": "anchor_decoder.mlp_feature_bank",
                "embedding_appearance": "embedding_appearance"}


def transform_gs_mlp_checkpoint(ckpt_path: str, out_dir: str = None, point_cloud: str = None) -> str:
    """Convert a decoder file of Scaffold-GS / Octree-GS - one state dict per head under ``opacity_mlp``, ``cov_mlp``,
    ``color_mlp`` (optionally ``mlp_feature_bank``, ``embedding_appearance``; an ``anchor_decoder.`` prefix on the keys
    is accepted) - into the flat ``state_dict.th`` the models load beside ``point_cloud.ply``.  The reference does this
    remapping by hand before its render tests (tests/test_module/test_util/test_gs_ckpt_transform.py:59-90).

    ``out_dir`` defaults to the folder of ``ckpt_path``; ``point_cloud`` (default: ``point_cloud.ply`` beside the
    input) is copied along when it exists and ``out_dir`` differs.  Returns the path of ``state_dict.th``."""
    import os
    import shutil

    heads = torch.load(ckpt_path, map_location="cpu", weights_only=False)
    flat = {}
    for key, sub in heads.items():
        short = key.split("anchor_decoder.", 1)[-1]
        if short in _GS_MLP_KEYS and isinstance(sub, dict):
            for name, value in sub.items():
                flat[f"{_GS_MLP_KEYS[short]}.{name}"] = value
    assert flat, f"{ckpt_path}: none of the decoder keys {sorted(_GS_MLP_KEYS)} found"
    src_dir = os.path.dirname(os.path.abspath(ckpt_path))
    out_dir = out_dir or src_dir
    os.makedirs(out_dir, exist_ok=True)
    ply = point_cloud or os.path.join(src_dir, "point_cloud.ply")
    if os.path.exists(ply) and os.path.abspath(out_dir) != os.path.dirname(os.path.abspath(ply)):
        shutil.copyfile(ply, os.path.join(out_dir, "point_cloud.ply"))
    out = os.path.join(out_dir, "state_dict.th")
    torch.save(flat, out)
    return out
