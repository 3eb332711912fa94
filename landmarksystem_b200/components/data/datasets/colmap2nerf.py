"""COLMAP reconstruction -> ``transforms_train.json`` / ``transforms_test.json``.

The reference's data-preparation page asks for this conversion (``colmap2nerf.py --recon_dir ... --output_dir ...``,
doc/source/quickstart.md:81-85) without shipping the script.  A sparse model (``cameras / images / points3D`` in binary
or text form) becomes the transforms layout every JSON dataset of this package reads: OpenGL camera-to-world matrices,
images addressed as ``./images/<name>``, one focal length for the whole file when all images share a camera and focal
length / size per frame otherwise.  Every ``holdout``-th image (sorted by name) goes to the test file.

    python -m landmarksystem_b200.components.data.datasets.colmap2nerf --recon_dir data/scene/sparse/0 --output_dir data/scene
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, List, Tuple

import numpy as np

from .colmap_loader import ColmapCamera, ColmapImage, read_model


def camera_to_world_opengl(image: ColmapImage) -> np.ndarray:
    """``[4, 4]`` camera-to-world matrix in OpenGL axes (x right, y up, z backward) of a COLMAP image record."""
    w2c = np.eye(4)
    w2c[:3, :3], w2c[:3, 3] = image.rotation(), image.tvec
    c2w = np.linalg.inv(w2c)
    c2w[:3, 1:3] *= -1.0
    return c2w


def _frame(image: ColmapImage, camera: ColmapCamera, image_dir: str, per_frame: bool) -> Dict:
    frame = {"file_path": f"./{image_dir}/{image.name}", "transform_matrix": camera_to_world_opengl(image).tolist()}
    if per_frame:
        fx, fy = camera.focal()
        frame.update(fl_x=fx, fl_y=fy, w=int(camera.width), h=int(camera.height))
    return frame


def convert(recon_dir: str, output_dir: str, holdout: int = 8, image_dir: str = "images") -> Tuple[int, int]:
    """Write the two transforms files into ``output_dir``; returns ``(n_train, n_test)``.  ``holdout <= 0`` keeps every
    image in the training file (the test file then repeats the first image so that evaluators have a view)."""
    cameras, images, _ = read_model(recon_dir)
    ordered: List[ColmapImage] = sorted(images.values(), key=lambda im: im.name)
    assert ordered, f"{recon_dir}: the model has no images"
    used = {im.camera_id for im in ordered}
    per_frame = len(used) > 1
    head: Dict = {"camera_model": "SIMPLE_PINHOLE"}
    if not per_frame:
        cam = cameras[next(iter(used))]
        fx, fy = cam.focal()
        head.update(fl_x=fx, fl_y=fy, w=int(cam.width), h=int(cam.height))
    train, test = [], []
    for k, im in enumerate(ordered):
        (test if holdout > 0 and k % holdout == 0 else train).append(_frame(im, cameras[im.camera_id], image_dir, per_frame))
    if not test:
        test = train[:1]
    os.makedirs(output_dir, exist_ok=True)
    for split, frames in (("train", train), ("test", test)):
        with open(os.path.join(output_dir, f"transforms_{split}.json"), "w", encoding="utf-8") as fh:
            json.dump(dict(head, frames=frames), fh, indent=1)
    return len(train), len(test)


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description="COLMAP sparse model -> transforms_train.json / transforms_test.json")
    parser.add_argument("--recon_dir", required=True, help="folder with cameras / images / points3D (.bin or .txt)")
    parser.add_argument("--output_dir", required=True)
    parser.add_argument("--holdout", type=int, default=8, help="every n-th image (by name) is a test view; 0: none")
    parser.add_argument("--image_dir", default="images", help="image folder relative to output_dir")
    args = parser.parse_args(argv)
    n_train, n_test = convert(args.recon_dir, args.output_dir, args.holdout, args.image_dir)
    print(f"wrote {n_train} training and {n_test} test frames to {args.output_dir}", flush=True)


if __name__ == "__main__":
    main()
