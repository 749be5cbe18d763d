from tokasaurus_b200.parts.base import (  # noqa: F401
    FeedForward,
    InputStage,
    Mixer,
    Norm,
    PagedCacheNeed,
    Part,
    PositionEncoding,
    QkvStage,
    ResidualStream,
    StateNeed,
    WeightSpec,
)
from tokasaurus_b200.parts.norm import GroupRMSNorm, LayerNorm, RMSNorm  # noqa: F401
from tokasaurus_b200.parts.conv import ShortConv  # noqa: F401
from tokasaurus_b200.parts.rope import NoPositionEncoding, RotaryEncoding, SinusoidalPositions  # noqa: F401
from tokasaurus_b200.parts.attention import PagedAttention  # noqa: F401
from tokasaurus_b200.parts.mlp import ClampedGLU, GatedMLP, PolyNormMLP, RoutedExperts  # noqa: F401
from tokasaurus_b200.parts.recurrent import (  # noqa: F401
    DecayedLinearAttention,
    GatedLinearAttention,
    GatedLinearRecurrence,
    Retention,
)
from tokasaurus_b200.parts.state_space import SelectiveStateSpace  # noqa: F401
from tokasaurus_b200.parts.sink_attention import SinkAttention  # noqa: F401
from tokasaurus_b200.parts.diff_attention import DifferentialAttention  # noqa: F401
from tokasaurus_b200.parts.latent_attention import LatentAttention  # noqa: F401
from tokasaurus_b200.parts.side_input import TokenSideInput  # noqa: F401
from tokasaurus_b200.parts.block import OutputNormBlock, PostNormBlock, PreNormBlock  # noqa: F401
from tokasaurus_b200.parts.embedding import OutputHead, TokenEmbedding  # noqa: F401
from tokasaurus_b200.parts.model import DecoderModel, LayerCall  # noqa: F401
