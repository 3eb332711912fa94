"""Dataset registries (reference: landmark/nerf_components/data/datasets/dataloader/__init__.py:8-17)."""
from .base_dataset import BaseDataset, GaussianSplattingDataset, VolumeRenderDataset
from .colmap_dataset import ColmapGaussianDataset, ZhangjiangGaussianDataset
from .json_datasets import BlenderDataset, CityDataset, CityGaussianDataset, MatrixCityDataset
from .synthetic_dataset import SyntheticGaussianDataset, SyntheticNeRFDataset

dataset_dict = {"city": CityDataset, "matrixcity": MatrixCityDataset, "blender": BlenderDataset,
                "synthetic": SyntheticNeRFDataset}
gaussian_dataset_dict = {"city": CityGaussianDataset, "matrixcity": CityGaussianDataset, "colmap": ColmapGaussianDataset, "Colmap": ColmapGaussianDataset,
                         "zhangjiang": ZhangjiangGaussianDataset, "synthetic": SyntheticGaussianDataset}

__all__ = ["BaseDataset", "GaussianSplattingDataset", "VolumeRenderDataset", "BlenderDataset", "CityDataset",
           "CityGaussianDataset", "ColmapGaussianDataset", "ZhangjiangGaussianDataset", "MatrixCityDataset", "SyntheticGaussianDataset", "SyntheticNeRFDataset",
           "dataset_dict", "gaussian_dataset_dict"]
