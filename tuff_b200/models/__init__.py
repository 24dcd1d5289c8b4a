from .model import Model
from .spec import LayerSpec, ModelSpec, ScheduleEntry

__all__ = ["Model", "ModelSpec", "LayerSpec", "ScheduleEntry"]
