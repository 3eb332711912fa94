"""Pydantic base for every typed configuration block
(reference: landmark/nerf_components/configs/base_configclass.py:6-23)."""
from pydantic import BaseModel, ConfigDict


class ConfigClass(BaseModel):
    """Typed config block. Unknown fields are ignored; arbitrary (tensor/device) types are allowed."""

    model_config = ConfigDict(arbitrary_types_allowed=True, extra="ignore", protected_namespaces=())

    def check_args(self) -> None:
        """Hook for cross-field validation; subclasses extend it."""
        return None
