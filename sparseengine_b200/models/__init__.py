"""Architecture builders.  Importing this package registers them."""
from . import bavutar, kisusun, minimax_m2, tedisun, zisevik  # noqa: F401
