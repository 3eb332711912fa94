"""Small enums shared by the rendering engine and the components (reference:
landmark/render/util/types.py:15-36)."""
from enum import Enum


class RuntimeType(str, Enum):
    Kernel = "Kernel"
    Torch = "Torch"


class MergeType(str, Enum):
    Evenly = "Evenly"      # equal chunks along a dimension
    Unevenly = "Unevenly"  # explicit split sizes along a dimension
    List = "List"          # one state-dict key per block

    @classmethod
    def check(cls, item) -> bool:
        """Whether ``item`` names a merge type (reference: landmark/render/util/types.py:20-26)."""
        try:
            cls(item)
        except ValueError:
            return False
        return True


class StageInput(str, Enum):
    Args = "Args"
    Kwargs = "Kwargs"
