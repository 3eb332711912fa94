"""Process environment: rank / world size discovery for torchrun and SLURM
(reference: landmark/utils/env.py:22-46)."""
from __future__ import annotations

import os
import subprocess


def parse_env(env_name: str) -> bool:
    """A boolean switch from the environment: ``True`` / ``ON`` / ``1`` are true, unset / ``False`` / ``OFF`` / ``0``
    false, anything else is an error (reference: landmark/utils/env.py:6-19)."""
    value = os.getenv(env_name)
    if value in ("True", "ON", "1"):
        return True
    if value in (None, "False", "OFF", "0"):
        return False
    raise NotImplementedError(f"{env_name}={value!r}: expected True/ON/1 or False/OFF/0")


def _slurm_master_addr() -> str:
    nodelist = os.environ.get("SLURM_NODELIST", "")
    try:
        out = subprocess.run(
            ["scontrol", "show", "hostnames", nodelist], capture_output=True, text=True, check=True
        ).stdout.split()
        return out[0] if out else "127.0.0.1"
    except (OSError, subprocess.CalledProcessError):
        return "127.0.0.1"


class EnvSetting:
    """Class-level constants read once at import; ``refresh`` re-reads the environment."""

    SLURM: bool = False
    COMM_TIMEOUT: int = 1800
    WORLD_SIZE: int = 1
    RANK: int = 0
    LOCAL_RANK: int = 0

    @classmethod
    def refresh(cls) -> None:
        env = os.environ
        cls.SLURM = "SLURM_PROCID" in env and "RANK" not in env
        cls.COMM_TIMEOUT = int(env.get("COMM_TIMEOUT", 1800))
        if cls.SLURM:
            cls.RANK = int(env["SLURM_PROCID"])
            cls.WORLD_SIZE = int(env.get("SLURM_NTASKS", 1))
            cls.LOCAL_RANK = int(env.get("SLURM_LOCALID", 0))
            env.setdefault("MASTER_ADDR", _slurm_master_addr())
            env.setdefault("MASTER_PORT", str(29500 + int(env.get("SLURM_JOB_ID", "0")) % 1000))
            env["RANK"], env["WORLD_SIZE"], env["LOCAL_RANK"] = str(cls.RANK), str(cls.WORLD_SIZE), str(cls.LOCAL_RANK)
        else:
            cls.RANK = int(env.get("RANK", 0))
            cls.WORLD_SIZE = int(env.get("WORLD_SIZE", 1))
            cls.LOCAL_RANK = int(env.get("LOCAL_RANK", cls.RANK))


EnvSetting.refresh()
