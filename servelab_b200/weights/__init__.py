"""Weights by tensor name: sources, checks, precision policy, random folders."""

from .random_init import write_random_model
from .safetensors_io import SafetensorsFile, write_safetensors
from .source import (BIAS, MATRIX, NORM, TABLE, FolderSource, RandomSource, TensorDecl,
                     WeightsError, WeightSource, check_source)
from .store import WeightStore

__all__ = ["BIAS", "MATRIX", "NORM", "TABLE", "FolderSource", "RandomSource",
           "SafetensorsFile", "TensorDecl", "WeightSource", "WeightStore",
           "WeightsError", "check_source", "write_random_model", "write_safetensors"]
