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
from .init import (XavierUniform, XavierNormal, KaimingUniform, KaimingNormal, Constant, ZerosInit, OnesInit,  # noqa
                   Uniform, Normal, Orthogonal)
from .module import NamedParameters  # noqa
from .loss import *  # noqa
from .loss import (MSELoss, MAELoss, L1Loss, HuberLoss, SmoothL1Loss, CrossEntropyLoss, NLLLoss, BCELoss,  # noqa
                   BCEWithLogitsLoss, KLDivLoss, PoissonNLLLoss, GaussianNLLLoss, MarginRankingLoss,
                   HingeEmbeddingLoss, CosineEmbeddingLoss, TripletMarginLoss, MultiMarginLoss, SoftMarginLoss,
                   MultiLabelSoftMarginLoss, MultiLabelMarginLoss, TripletMarginWithDistanceLoss, CTCLoss,
                   PairwiseL2Distance)
from .conv import (Conv1d, Conv2d, Conv3d, ConvTranspose1d, ConvTranspose2d, ConvTranspose3d, Unfold, Fold)  # noqa
from .pool import *  # noqa
from .batchnorm import (BatchNorm1d, BatchNorm2d, BatchNorm3d, GroupNorm, InstanceNorm1d, InstanceNorm2d,  # noqa
                        InstanceNorm3d, LocalResponseNorm)
from .shape_layers import *  # noqa
from .rnn import (RNNCell, LSTMCell, GRUCell, RNN, LSTM, GRU, Seq2Seq, PackedSequence, PadSequence,  # noqa
                  UnpadSequence, PackPaddedSequence, PackSequence, PadPackedSequence)
from .adaptive_softmax import AdaptiveLogSoftmaxWithLoss  # noqa
from .hooks import (RegisterForwardPreHook, RegisterForwardHook, RegisterFullBackwardHook, RemoveHook,  # noqa
                    RegisterModuleForwardPreHook, RegisterModuleForwardHook, RegisterModuleFullBackwardHook,
                    RemoveModuleHook, Call)
from .stateless import (WithReplacedParams, FunctionalCall, FunctionalCallMulti, FunctionalCallGrad,  # noqa
                        FunctionalCallGradMulti, WithGradsToReplacements)
from .lazy import *  # noqa
from .lazy import IsLazy  # noqa
from .fuse import FuseConvBNEval, FuseLinearBNEval  # noqa
from .parametrize import *  # noqa
from . import prune  # noqa
from .types import *  # noqa


from ..options import accepting_options as _accepting_options, package_getattr as _package_getattr


def _constructor_aliases(ns) -> None:
    """``NewX`` for every public class ``X``: the reference builds modules with constructor
    functions (``nn.NewLinear(3, 4)``, ``nn.NewConv2d(3, 16, 3, nn.WithPadding(1))``).  Each
    ``NewX`` calls ``X`` after turning option objects into keyword arguments; the loss functions
    accept options the same way (``nn.CrossEntropyLoss(z, y, nn.WithLabelSmoothing(0.1))``)."""
    for name, obj in list(ns.items()):
        if (isinstance(obj, type) or name.startswith("Lazy")) and name[0].isupper() and "New" + name not in ns:
            ns["New" + name] = _accepting_options(obj)
        elif callable(obj) and not isinstance(obj, type) and name.endswith("Loss") and name[0].isupper():
            ns[name] = _accepting_options(obj)


def NewSequential(*layers):
    return Sequential(*layers)  # noqa: F405


def NewModuleList(*mods):
    """Variadic, as in the reference (nn/containers.go:27-40); one list is accepted too."""
    return ModuleList(list(mods[0]) if len(mods) == 1 and isinstance(mods[0], (list, tuple)) else list(mods))  # noqa: F405


def NewParameterList(*ps):
    return ParameterList(list(ps[0]) if len(ps) == 1 and isinstance(ps[0], (list, tuple)) else list(ps))  # noqa: F405


def NewUnflatten(dim, *sizes):
    return Unflatten(dim, tuple(sizes[0]) if len(sizes) == 1 and isinstance(sizes[0], (list, tuple)) else sizes)  # noqa: F405


_constructor_aliases(globals())
__getattr__ = _package_getattr(__name__)     # nn.WithPadding(1), nn.WithBidirectional(), ...


def NewLayerNormShape(shape, **kw):
    """LayerNorm over several trailing dimensions (nn/norm.go:104-113)."""
    return LayerNorm(tuple(shape), **kw)  # noqa: F405
