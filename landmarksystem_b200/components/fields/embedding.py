"""Per-image appearance embedding (reference:
landmark/nerf_components/model_components/fields/embedding.py:5-46)."""
import torch


class AppearanceEmbedding(torch.nn.Module):
    def __init__(self, n_imgs: int, n_component: int, device) -> None:
        super().__init__()
        self.device = device
        self.embedding = torch.nn.Embedding(n_imgs, n_component, device=device)

    def forward(self, idxs=None, xyz_sampled=None, app_code=None):
        if idxs is not None:
            return self.embedding(idxs.long())
        if app_code is not None:
            code = torch.as_tensor(app_code, device=self.embedding.weight.device).long()
            return self.embedding(code.expand(xyz_sampled.shape[:-1]))
        return None
