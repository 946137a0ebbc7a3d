from . import bosenex, gpt2, pidodra, zirunex, zudalorn  # noqa: F401
from .decoder import DecoderModel, ModelSpec, ScheduleEntry
from .loading import load_model

__all__ = ["DecoderModel", "ModelSpec", "ScheduleEntry", "load_model"]
