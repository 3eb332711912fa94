from .convertor_factory import ComponentConvertorFactory, ParallelConvertor, RuntimeConvertor

__all__ = ["ComponentConvertorFactory", "ParallelConvertor", "RuntimeConvertor"]
