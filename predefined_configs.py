"""`from predefined_configs import get_config` as in the reference's scripts."""
from state_space_models_neuron_b200.models.predefined_configs import (CONFIGS_KWARGS, ConfParams,  # noqa: F401
                                                                      MAMBA2_CONFIGS_KWARGS,
                                                                      MAMBA2HYBRID_CONFIGS_KWARGS, get_config)
