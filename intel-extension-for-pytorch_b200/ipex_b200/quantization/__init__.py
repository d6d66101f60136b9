from ._qconfig import (  # noqa: F401
    QConfigWoq,
    WoqActQuantMode,
    WoqLowpMode,
    WoqWeightDtype,
    WoqWeightQScheme,
    get_weight_only_quant_qconfig_mapping,
)
from ._quantize_utils import (  # noqa: F401
    dequantize_per_block,
    dequantize_per_channel,
    quantize_per_block,
    quantize_per_channel,
)
