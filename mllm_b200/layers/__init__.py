from .attention import RadixAttention
from .embedding import VocabParallelEmbedding
from .linear import ColumnParallelLinear, Linear, MergedLinear, RowParallelLinear
from .mlp import MLP, ParallelMLP
from .norm import GemmaRMSNorm, LayerNorm, RMSNorm
from .quantize_base import LinearMethodBase, QuantizeMethodBase, UnquantizedLinearMethod, set_weight_attrs
