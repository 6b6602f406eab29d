"""Reference model families used by the benchmarks and tests: Llama-style decoder, Mixtral-style MoE
decoder and ResNet-50, written against stock ``torch.nn`` plus the backend's fused operators."""
from .llama import LlamaConfig, Llama, llama_7b_config, llama_tiny_config  # noqa: F401
from .moe import MoEConfig, MoETransformer, moe_tiny_config  # noqa: F401,E402
from . import resnet  # noqa: F401,E402
from .resnet import ResNet, resnet18, resnet50  # noqa: F401,E402


def _install_fused_bn():
    from ..ops.modules import bn_module_act

    resnet.FUSED_BN_ACT = bn_module_act


_install_fused_bn()
