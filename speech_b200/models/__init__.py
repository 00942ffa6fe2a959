"""Model classes (the public entry points users instantiate or restore)."""
from .ctc_models import EncDecCTCModel, EncDecCTCModelBPE  # noqa: F401
from .hybrid_models import EncDecHybridRNNTCTCBPEModel, EncDecHybridRNNTCTCModel  # noqa: F401
from .rnnt_models import EncDecRNNTBPEModel, EncDecRNNTModel  # noqa: F401
from .aed_models import EncDecMultiTaskModel  # noqa: F401
