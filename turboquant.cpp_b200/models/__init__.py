"""Models: the generic decoder and the architectures built on it."""
from .decoder import DecoderModel, Embedding, LMHead, PairEmbedding, ScheduleEntry
from .qwen2_moe import Qwen2MoeModel
from .nuforax import NuforaxModel
from .lumevik import LumevikModel
from .sisepel import SisepelModel
from .tasadra import TasadraModel
