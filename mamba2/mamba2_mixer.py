from state_space_models_neuron_b200.models.cache import Mamba2Cache  # noqa: F401
from state_space_models_neuron_b200.models.mamba2_mixer import (DepthwiseConv1d, Mamba2Mixer,  # noqa: F401
                                                                MambaRMSNormGated)
