from .decoder import Decoder, ModelSpec, LayerCall, CacheGroup
from . import llama, kavenex, murilorn, luvapel, midulorn
