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
