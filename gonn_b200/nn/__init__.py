"""Layer catalogue."""
from .module import (Module, Sequential, ModuleList, ModuleDict, ParameterList, ParameterDict, Identity,  # noqa
                     Flatten, Unflatten, FilterParams, filter_params)
from .linear import Linear, Bilinear  # noqa
from .norm import LayerNorm, RMSNorm  # noqa
from .activation import *  # noqa
from .embedding import Embedding, EmbeddingBag  # noqa
from .dropout import Dropout, Dropout1d, Dropout2d, Dropout3d, AlphaDropout, FeatureAlphaDropout  # noqa
from .attention import MultiHeadAttention  # noqa
from .transformer import (TransformerEncoderLayer, TransformerEncoder, TransformerDecoderLayer,  # noqa
                          TransformerDecoder, Transformer)
from . import init  # noqa
from .loss import *  # noqa
from .loss import (MSELoss, MAELoss, L1Loss, HuberLoss, SmoothL1Loss, CrossEntropyLoss, NLLLoss, BCELoss,  # noqa
                   BCEWithLogitsLoss, KLDivLoss, PoissonNLLLoss, GaussianNLLLoss, MarginRankingLoss,
                   HingeEmbeddingLoss, CosineEmbeddingLoss, TripletMarginLoss, MultiMarginLoss, SoftMarginLoss,
                   MultiLabelSoftMarginLoss, MultiLabelMarginLoss, TripletMarginWithDistanceLoss, CTCLoss,
                   PairwiseL2Distance)
