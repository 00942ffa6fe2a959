"""Model classes (the public entry points users instantiate or restore)."""
from .aed_models import EncDecMultiTaskModel  # noqa: F401
from .asr_variants import (  # noqa: F401
    ConfidenceEnsembleModel,
    EncDecHybridRNNTCTCBPEEOUModel,
    EncDecHybridRNNTCTCBPEModelWithPrompt,
    EncDecMultiTalkerRNNTBPEModel,
    EncDecRNNTBPEEOUModel,
    EncDecRNNTBPEModelWithPrompt,
)
from .classification_models import (  # noqa: F401
    EncDecClassificationModel,
    EncDecFrameClassificationModel,
    EncDecRegressionModel,
    EncDecSpeakerLabelModel,
)
from .ctc_models import EncDecCTCModel, EncDecCTCModelBPE  # noqa: F401
from .diarizers import ClusteringDiarizer, OnlineDiarizer  # noqa: F401
from .hybrid_models import EncDecHybridRNNTCTCBPEModel, EncDecHybridRNNTCTCModel  # noqa: F401
from .rnnt_models import EncDecRNNTBPEModel, EncDecRNNTModel  # noqa: F401
from .sortformer_models import SortformerEncLabelModel  # noqa: F401
from .transformer_bpe_models import EncDecTransfModelBPE  # noqa: F401
from .ssl_models import (  # noqa: F401
    EncDecDenoiseMaskedTokenPredModel,
    EncDecMaskedTokenPredModel,
    SpeechEncDecSelfSupervisedModel,
)
