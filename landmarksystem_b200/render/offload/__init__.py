"""Dynamic loading of scene blocks (reference: landmark/render/parameter_loader/__init__.py exports ``OffloadModule``);
resolved on first access because the module imports the inference stack."""


def __getattr__(name):
    if name == "OffloadModule":
        from .offload_module import OffloadModule

        return OffloadModule
    raise AttributeError(name)


__all__ = ["OffloadModule"]
