from .base_sampler import BaseSampler
from .pdf_sampler import PDFSampler, sample_pdf
from .uniform_sampler import FusedUniformSampler, UniformSampler

__all__ = ["BaseSampler", "PDFSampler", "sample_pdf", "UniformSampler", "FusedUniformSampler"]
