"""Import-path compatibility: `mamba2hybrid.*` of the reference maps onto the framework package."""
from state_space_models_neuron_b200.models import (Mamba2HybridConfig, Mamba2HybridForCausalLM,  # noqa: F401
                                                   Mamba2HybridModel, allocate_layers)
