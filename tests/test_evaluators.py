"""Train briefly, then evaluate from the checkpoint through the evaluator entry points."""
import os

import numpy as np
import pytest

from landmarksystem_b200.configs import BaseConfig

ROOT = os.path.join(os.path.dirname(__file__), "..", "landmarksystem_b200", "models")
CASES = [("gridnerf", "gridnerf_trainer", "GridNeRFTrainer", "gridnerf_evaluator", "GridNeRFEvaluator", "synthetic_tiny.py", {"nSamples": "24"}),
         ("instant_ngp", "instant_ngp_trainer", "NGPTrainer", "instant_ngp_evaluator", "NGPEvaluator", "synthetic_tiny.py", {}),
         ("nerfacto", "nerfacto_trainer", "NerfactoTrainer", "nerfacto_evaluator", "NerfactoEvaluator", "synthetic_tiny.py", {}),
         ("origin_gs", "gs_trainer", "Gaussian3DTrainer", "gs_evaluator", "Gaussian3DEvaluator", "synthetic_train.py", {"init_points_num": "60"}),
         ("scaffold_gs", "gs_trainer", "ScaffoldGSTrainer", "gs_evaluator", "ScaffoldGSEvaluator", "synthetic_train.py", {"init_points_num": "60"}),
         ("octree_gs", "gs_trainer", "OctreeGSTrainer", "gs_evaluator", "OctreeGSEvaluator", "synthetic_train.py", {"init_points_num": "60"})]


@pytest.mark.parametrize("family,tmod,tcls,emod,ecls,conf,extra", CASES)
def test_train_then_evaluate_cpu(family, tmod, tcls, emod, ecls, conf, extra, tmp_path):
    import importlib

    over = {"basedir": str(tmp_path), "device": "cpu", "n_iters": "3", "datadir": "ring:3:12x12:14:3", "batch_size": "64",
            "progress_refresh_rate": "100", "N_vis": "-1"}
    over.update(extra)
    gaussian = family.endswith("_gs")
    if gaussian:
        over["batch_size"] = "1"
    path = os.path.join(ROOT, family, "confs", conf)
    trainer = getattr(importlib.import_module(f"landmarksystem_b200.models.{family}.{tmod}"), tcls)(BaseConfig.from_file(path, over))
    trainer.train()
    assert np.isfinite(trainer.eval())
    cfg = BaseConfig.from_file(path, over)
    cfg.is_train = False
    cfg.ckpt = (os.path.join(trainer.logfolder, "point_cloud", "iteration_3", "point_cloud.ply") if gaussian
                else os.path.join(trainer.logfolder, "state_dict.th"))
    if family == "instant_ngp":                  # "auto": the files of the run with this experiment name
        cfg.ckpt = "auto"
    ev = getattr(importlib.import_module(f"landmarksystem_b200.models.{family}.{emod}"), ecls)(cfg)
    assert np.isfinite(ev.eval())
    if family == "instant_ngp":
        assert ev.config.ckpt == os.path.join(trainer.logfolder, "state_dict.th")
    assert any(f.endswith(".png") for f in os.listdir(ev.save_folder))
    if family == "gridnerf":                     # the "path" split: a fly-around without ground truth
        cfg.render_spherical, cfg.render_nframes, cfg.render_px = True, 3, 9
        cfg.render_spherical_radius, cfg.render_near_far = 3.0, None
        assert ev.render_path() == 3
        frames = sorted(f for f in os.listdir(os.path.join(ev.logfolder, "imgs_path_all")) if f.startswith("path_"))
        assert len(frames) == 3


def test_command_line_entry_points_train_evaluate_and_render_a_path(tmp_path):
    """``python -m ...gridnerf_trainer --config ... --key value`` then ``...gridnerf_evaluator --ckpt auto --render_path
    True``: console overrides (also of fields the file leaves unset), checkpoint discovery by experiment name, test
    views and a fly-around written by one evaluator call."""
    import glob

    from landmarksystem_b200.models.gridnerf import gridnerf_evaluator, gridnerf_trainer

    conf = os.path.join(ROOT, "gridnerf", "confs", "synthetic_tiny.py")
    common = ["--config", conf, "--basedir", str(tmp_path), "--device", "cpu", "--datadir", "ring:3:12x12:14:3",
              "--batch_size", "64", "--nSamples", "24", "--N_vis", "-1"]
    gridnerf_trainer.main(common + ["--n_iters", "3", "--progress_refresh_rate", "100"])
    run = glob.glob(str(tmp_path / "*"))[0]
    gridnerf_evaluator.main(common + ["--ckpt", "auto", "--render_path", "True", "--render_spherical", "True",
                                      "--render_nframes", "2", "--render_px", "9", "--render_spherical_radius", "3.0"])
    assert sorted(os.listdir(os.path.join(run, "imgs_path_all"))) == ["path_000.png", "path_001.png"]
    assert any(f.endswith(".png") for f in os.listdir(os.path.join(run, "imgs_test_all")))
