from .decoder import DecoderModel, decoder_param_specs
from . import gemma3 as _gemma3      # registers the architecture
from . import ramilorn as _ramilorn  # registers the architecture
from . import zazerax as _zazerax    # registers the architecture
from . import bovozen as _bovozen    # registers the architecture
from . import kadavik as _kadavik    # registers the architecture

__all__ = ["DecoderModel", "decoder_param_specs"]
