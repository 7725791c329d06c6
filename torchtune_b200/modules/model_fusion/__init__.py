from ._layers import FusionEmbedding, FusionLayer, get_fusion_params, register_fusion_module
from ._models import DeepFusionModel, EarlyFusionModel

__all__ = ["DeepFusionModel", "EarlyFusionModel", "FusionEmbedding", "FusionLayer", "get_fusion_params", "register_fusion_module"]
