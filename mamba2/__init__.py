"""Import-path compatibility: `mamba2.*` of the reference maps onto the framework package."""
from state_space_models_neuron_b200.models import (Mamba2Cache, Mamba2Config, Mamba2ForCausalLM,  # noqa: F401
                                                   Mamba2Mixer, Mamba2Model)
