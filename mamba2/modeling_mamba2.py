from state_space_models_neuron_b200.models.modeling_mamba2 import *  # noqa: F401,F403
from state_space_models_neuron_b200.models.modeling_mamba2 import (Mamba2Block, Mamba2CausalLMOutput,  # noqa: F401
                                                                   Mamba2ForCausalLM, Mamba2Model, Mamba2Output,
                                                                   Mamba2PreTrainedModel, Mamba2RMSNorm)
