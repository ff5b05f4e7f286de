"""Drop-in import name of the reference package: `import teramoe` resolves to teramoe_b200."""
from teramoe_b200 import *  # noqa: F401,F403
from teramoe_b200 import Buffer, Config, EventOverlap, AutotuneResult, autotune_teramoe, topk_idx_t  # noqa: F401
