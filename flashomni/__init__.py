"""Drop-in name for the reference's package: `import flashomni` gives the same public surface the reference's
`flashomni/__init__.py` exports (`BatchFlashOmniFAWithRaggedKVWrapper`, `flashomni_gemm`,
`flashomni_gemm_reduction`, `packbits`, `segment_packbits`, `__version__`) and the same submodules
(`flashomni.attention`, `flashomni.gemm`, `flashomni.quantization`, `flashomni.utils`), all served by
flashomni_b200. Scripts written against the reference run unchanged with this directory's parent on sys.path."""

from flashomni_b200 import __version__ as __version__
from . import attention as attention
from . import gemm as gemm
from . import quantization as quantization
from . import utils as utils
from .attention import *  # noqa: F401,F403
from .gemm import flashomni_gemm as flashomni_gemm
from .gemm import flashomni_gemm_reduction as flashomni_gemm_reduction
from .quantization import packbits as packbits
from .quantization import segment_packbits as segment_packbits
