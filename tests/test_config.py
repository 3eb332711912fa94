"""L0: attribute dict, typed config blocks, conf-file loading and console overrides."""
import os
import textwrap

import pytest

from landmarksystem_b200.configs import BaseConfig, DatasetConfig, RenderConfig, TrainConfig, parse_console_args
from landmarksystem_b200.utils import Config, SingletonMeta


def test_config_attr_access_and_nesting():
    c = Config({"a": 1, "b": {"c": 2}})
    assert c.a == 1 and c.b.c == 2 and isinstance(c.b, Config)
    c.d = {"e": 3}
    assert c["d"].e == 3
    assert not hasattr(c, "missing")
    assert c.to_dict() == {"a": 1, "b": {"c": 2}, "d": {"e": 3}}


def test_config_from_file_skips_modules_and_classes(tmp_path):
    f = tmp_path / "x.py"
    f.write_text("import os\nclass K: pass\nvalue = 5\nnested = dict(k=1)\n")
    c = Config.from_file(f)
    assert c.value == 5 and c.nested.k == 1 and "os" not in c and "K" not in c


def test_singleton_meta():
    class S(metaclass=SingletonMeta):
        pass

    assert S() is S()


def test_parse_console_args():
    assert parse_console_args(["--a", "1", "--flag", "--b", "x"]) == {"a": "1", "flag": True, "b": "x"}
    assert parse_console_args(None) is None


def _write_conf(tmp_path, extra=""):
    conf = tmp_path / "conf.py"
    conf.write_text(textwrap.dedent(f"""
        from landmarksystem_b200.configs import DatasetConfig, TrainConfig
        t = TrainConfig(model_name="m", expname="e", n_iters=10, batch_size=128)
        d = DatasetConfig(datadir="ring", lb=[0, 0, 0], ub=[1, 1, 1])
        config = [t, d]
        {extra}
    """))
    return conf


def test_from_file_flattens_and_overrides(tmp_path):
    cfg = BaseConfig.from_file(_write_conf(tmp_path), {"n_iters": "25", "DDP": "true", "basedir": "/tmp/x"})
    assert cfg.n_iters == 25 and cfg.DDP is True and cfg.basedir == "/tmp/x"
    assert cfg.batch_size == 128 and cfg.datadir == "ring" and cfg.plane_division == [1, 1]


def test_from_file_rejects_unknown_and_non_scalar(tmp_path):
    conf = _write_conf(tmp_path)
    with pytest.raises(AssertionError):
        BaseConfig.from_file(conf, {"nope": "1"})
    with pytest.raises(AssertionError):
        BaseConfig.from_file(conf, {"plane_division": "[2,2]"})
    with pytest.raises(ValueError):
        BaseConfig.from_file(conf, {"DDP": "maybe"})


def test_duplicate_fields_rejected(tmp_path):
    conf = _write_conf(tmp_path, extra='config.append(TrainConfig(model_name="m", expname="e", n_iters=1))')
    with pytest.raises(AssertionError):
        BaseConfig.from_file(conf)


def test_save_config_roundtrip(tmp_path):
    cfg = BaseConfig.from_file(_write_conf(tmp_path))
    out = tmp_path / "dump.txt"
    cfg.save_config(out)
    lines = out.read_text().splitlines()
    assert lines == sorted(lines) and any(l.startswith("batch_size = 128") for l in lines)


def test_render_config_inherits_and_checks():
    t = TrainConfig(model_name="m", expname="e", n_iters=1, plane_division=[2, 2])
    r = RenderConfig().from_train_config(t)
    assert r.model_name == "m" and r.plane_division == [2, 2]
    r.check_args()
    with pytest.raises(AssertionError):
        RenderConfig(is_train=True).check_args()


def test_dataset_config_checks():
    with pytest.raises(AssertionError):
        DatasetConfig(datadir="x", lb=[0, 0], ub=[1, 1, 1]).check_args()
    with pytest.raises(AssertionError):
        DatasetConfig(datadir="x", dynamic_load=True, dataset_type="nerf").check_args()
    with pytest.raises(AssertionError):
        TrainConfig(model_name="m", expname="e", n_iters=1, channel_parallel=True, branch_parallel=True).check_args()


def test_every_shipped_configuration_loads():
    """Each model family ships the MatrixCity train / render variants (single, DDP, branch / channel parallel and
    the cross-layout render configurations); every file must parse into a merged, validated configuration."""
    import glob
    import os

    from landmarksystem_b200.configs import BaseConfig

    root = os.path.join(os.path.dirname(__file__), "..", "landmarksystem_b200", "models")
    files = sorted(glob.glob(os.path.join(root, "*", "confs", "matrixcity_*.py")))
    assert len(files) >= 60
    seen = {}
    for f in files:
        cfg = BaseConfig.from_file(f, {})
        seen[os.path.relpath(f, root)] = cfg
        assert cfg.get("expname") and cfg.get("model_name")
        if f.endswith("render.py"):
            assert not cfg.is_train and cfg.get("ckpt")
    bp = seen[os.path.join("gridnerf", "confs", "matrixcity_2block_multi_BranchParallel_10x5.py")]
    assert bp.branch_parallel and list(bp.plane_division) == [10, 5] and bp.ub[0] > 40
    b2c = seen[os.path.join("gridnerf", "confs", "matrixcity_2block_lowquality_Branch2ChannelParallel_render.py")]
    assert b2c.channel_parallel and b2c.channel_parallel_size == 2 and not b2c.branch_parallel and b2c.sampling_opt


def test_init_distributed_mode_reads_the_launcher_environment(monkeypatch):
    from landmarksystem_b200.train.utils import init_distributed_mode

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    assert init_distributed_mode("single_node") == {"rank": 0, "world_size": 1, "local_rank": 0}
    monkeypatch.setenv("SLURM_PROCID", "0"); monkeypatch.setenv("SLURM_NTASKS", "1"); monkeypatch.setenv("SLURM_LOCALID", "0")
    monkeypatch.setenv("SLURM_NODELIST", "gpu[017-020],gpu033")
    monkeypatch.delenv("MASTER_ADDR", raising=False)
    out = init_distributed_mode("slurm")
    import os

    assert out["world_size"] == 1 and os.environ["MASTER_ADDR"] == "gpu017"


def test_metrics_logger_with_wandb_flag_but_no_package(tmp_path, capsys):
    from landmarksystem_b200.utils.metrics import MetricsLogger

    log = MetricsLogger(str(tmp_path), wandb=True, run_name="t")
    log.log(1, {"Train/Loss": 0.5})
    log.close()
    assert (tmp_path / "metrics.jsonl").read_text().count("Train/Loss") == 1


def test_nerfacto_config_accepts_both_spellings_and_render_fields():
    """The reference spells two fields ``appearance_embed_dim`` / ``lr`` (nerfacto.py:47, 95); both spellings read the
    same value, and the ``render_*`` fields of the path split are part of the block."""
    from landmarksystem_b200.models.nerfacto.nerfacto import NerfactoConfig

    a = NerfactoConfig(appearance_embed_dim=8, lr=3e-3, render_px=360, render_spherical=True)
    assert a.appearance_embedding_dim == 8 and a.appearance_embed_dim == 8
    assert a.lr_init == 3e-3 and a.lr == 3e-3 and a.render_px == 360 and a.render_spherical
    b = NerfactoConfig(appearance_embedding_dim=16, lr_init=1e-3)
    assert b.appearance_embed_dim == 16 and b.lr == 1e-3
    flat = dict(iter(b))
    assert {"render_nframes", "render_pathid", "render_lb", "distance_scale", "render_stratified_sampling"} <= set(flat)


def test_package_root_exports_match_the_reference():
    """``landmark/__init__.py:4-19`` exports these names from the package root."""
    import landmarksystem_b200 as lm
    from landmarksystem_b200.components.model.base_model import Model
    from landmarksystem_b200.render.inference_module import InferenceModule

    assert lm.InferenceModule is InferenceModule and lm.Model is Model
    for name in ("InferenceEngine", "InferenceInterface", "InferenceModuleInitializer", "init_communication_context",
                 "init_inference", "Config", "EnvSetting"):
        assert getattr(lm, name) is not None
    with pytest.raises(AttributeError):
        lm.no_such_name


def test_env_switch_parsing_and_slurm_discovery(monkeypatch):
    """``parse_env`` and the SLURM branch of ``EnvSetting`` (reference: landmark/utils/env.py:6-46)."""
    from landmarksystem_b200.utils import EnvSetting, parse_env

    monkeypatch.delenv("LMB_TEST_SWITCH", raising=False)
    assert parse_env("LMB_TEST_SWITCH") is False
    for text, want in (("ON", True), ("1", True), ("True", True), ("OFF", False), ("0", False), ("False", False)):
        monkeypatch.setenv("LMB_TEST_SWITCH", text)
        assert parse_env("LMB_TEST_SWITCH") is want
    monkeypatch.setenv("LMB_TEST_SWITCH", "maybe")
    with pytest.raises(NotImplementedError):
        parse_env("LMB_TEST_SWITCH")

    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        monkeypatch.delenv(name, raising=False)
    monkeypatch.setenv("SLURM_PROCID", "5")
    monkeypatch.setenv("SLURM_NTASKS", "16")
    monkeypatch.setenv("SLURM_LOCALID", "1")
    monkeypatch.setenv("SLURM_JOB_ID", "4321")
    monkeypatch.setenv("SLURM_NODELIST", "node[01-02]")
    monkeypatch.setenv("COMM_TIMEOUT", "77")
    try:
        EnvSetting.refresh()
        assert EnvSetting.SLURM and (EnvSetting.RANK, EnvSetting.WORLD_SIZE, EnvSetting.LOCAL_RANK) == (5, 16, 1)
        assert EnvSetting.COMM_TIMEOUT == 77 and os.environ["MASTER_PORT"] == str(29500 + 321)
        assert os.environ["MASTER_ADDR"]                      # first host of the node list, or loopback without scontrol
    finally:
        for name in ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID", "SLURM_JOB_ID", "SLURM_NODELIST", "COMM_TIMEOUT",
                     "RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
            monkeypatch.delenv(name, raising=False)
        EnvSetting.refresh()
    assert not EnvSetting.SLURM and EnvSetting.WORLD_SIZE == 1


def test_console_override_of_a_field_the_file_leaves_unset(tmp_path):
    conf = tmp_path / "conf.py"
    conf.write_text(textwrap.dedent("""
        from landmarksystem_b200.configs import DatasetConfig, TrainConfig
        config = [TrainConfig(model_name="m", expname="x", n_iters=1), DatasetConfig(datadir="d", lb=[0, 0, 0], ub=[1, 1, 1])]
    """))
    assert BaseConfig.from_file(str(conf)).ckpt is None
    cfg = BaseConfig.from_file(str(conf), parse_console_args(["--ckpt", "log/x/state_dict.th"]))
    assert cfg.ckpt == "log/x/state_dict.th"
    assert BaseConfig.from_file(str(conf), {"ckpt": "none"}).ckpt is None
    assert BaseConfig.from_file(str(conf), {"ckpt": "12"}).ckpt == 12
