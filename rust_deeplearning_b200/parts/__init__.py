"""Parts of a model.  Importing the package registers the built-in kinds."""
from . import (attention, decay_attention, delta_rule, feed_forward, latent_attention, mixer_pair, model, norm,  # noqa: F401
               position, routed_experts, state_space)
