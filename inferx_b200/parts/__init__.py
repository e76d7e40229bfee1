# importing a module registers the kinds it defines
from . import (attention, embedding, feed_forward, latent_attention,  # noqa: F401
               linear_recurrence, norm, position, state_space, token_shift)
from .base import (BuildContext, GroupView, LayerCache, PagedKvNeed, StateNeed,  # noqa: F401
                   StepContext)
from .block import Block, DecoderModel  # noqa: F401
from .registry import build_part, known, register_part, unregister_part  # noqa: F401
from .specs import (ClampedGluSpec, GroupedRmsNormSpec,  # noqa: F401
                    InterleavedRopeSpec, LatentAttentionSpec, TokenShiftSpec)
from .specs import (AttentionSpec, LayerSpec, ModelSpec, MoeSpec, RmsNormSpec,  # noqa: F401
                    RopeSpec, RunEntry, SwiGluSpec)
