"""Operations beyond ``torch.distributed``'s set, under the module path the reference gives them
(``torchcomms.distwrap.collectives_extension``); they are defined in the package's ``__init__``."""
from . import new_window, reduce_scatter_quantized  # noqa: F401
