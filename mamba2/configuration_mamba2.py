from state_space_models_neuron_b200.models.configuration_mamba2 import Mamba2Config  # noqa: F401
