from .scene import (BlobField, SyntheticNeRFData, aerial_cameras, camera_rays, look_at, make_blob_dataset,
                    ring_cameras)

__all__ = ["BlobField", "SyntheticNeRFData", "aerial_cameras", "camera_rays", "look_at", "make_blob_dataset",
           "ring_cameras"]
