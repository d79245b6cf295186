from .cache import Mamba2Cache  # noqa: F401
from .configuration_mamba2 import Mamba2Config  # noqa: F401
from .configuration_mamba2hybrid import Mamba2HybridConfig  # noqa: F401
from .layer_allocation import allocate_layers  # noqa: F401
from .modeling_mamba2 import (Mamba2Block, Mamba2CausalLMOutput, Mamba2ForCausalLM, Mamba2Model,  # noqa: F401
                              Mamba2Output, Mamba2PreTrainedModel, Mamba2RMSNorm)
from .mamba2_mixer import Mamba2Mixer, MambaRMSNormGated  # noqa: F401
from .predefined_configs import CONFIGS_KWARGS, ConfParams, get_config  # noqa: F401
from .hybrid_attn import Mamba2HybridAttention  # noqa: F401
from .hybrid_mlp import Mamba2HybridMLP  # noqa: F401
from .modeling_mamba2hybrid import (Mamba2HybridBlock, Mamba2HybridForCausalLM, Mamba2HybridModel,  # noqa: F401
                                    Mamba2HybridPreTrainedModel)
