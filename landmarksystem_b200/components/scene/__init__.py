from .scene_manager import SceneManager
