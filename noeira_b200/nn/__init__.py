from .arena import PARAM_ALIGN, ParamArena  # noqa: F401
from .combinators import (Checkpointed, Parallel, ProjectedResidual, Repeat, RepeatConditional, Residual,  # noqa: F401
                          Sequential, SkipConcat, StochasticActor, StopGradParams, Tokenwise)
from .init import (Constant, Deterministic, Kaiming, Normal, Orthogonal, ScaledKaiming, TruncNormalIn, Xavier,  # noqa: F401
                   Zero)
from .layers import (BiasAdd, Dropout, advance_rng, rng_step_counter, Elementwise, GaussianHead, Linear, LinearGELU, LinearReLU, LinearTanh,  # noqa: F401
                     Scale)
from .module import Module, apply, as_autograd, manual_seed  # noqa: F401
from .optim import SGD, Adam, AdamW, LaProp, ScalarAdam, polyak  # noqa: F401
from .param import Param, State  # noqa: F401
from .transformer import (AttentionCore, CrossAttention, Embedding, FeedForward, LayerNorm, MSELoss, RMSNorm,  # noqa: F401
                          SelfAttention, SwiGLU, SwiGLUFFN, TransformerBlock, cross_entropy, rope_, sincos_embed)
from .conv import (AvgPool2D, BasicBlock, BatchNorm2D, Conv2D, Conv2DTranspose, MaxPool2D, ResNet18Backbone, Upsample2D,  # noqa: F401
                   normalize_images)
from .graph import (ComputeGraph, ExternalNode, FusionReport, GraphExporter, InputSlot, MermaidExporter, Node,  # noqa: F401
                    TextExporter)
from . import schedulers  # noqa: F401
from .peft import (LoRALinear, QLinear, QLoRALinear, add_lora, dequantize_q4_0, freeze_params, quantize_linears,  # noqa: F401
                   quantize_q4_0, replace_linears)
from .recurrent import GRUCell, LSTMCell, LSTMSeq  # noqa: F401
from . import losses  # noqa: F401
from .noisy import BlockLinear, NoisyLinear, reset_noise  # noqa: F401
