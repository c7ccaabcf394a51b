from daser_b200.position.base import PositionEncoder  # noqa: F401
from daser_b200.position.fixed_offset import FixedOffsetEncoder  # noqa: F401
from daser_b200.position.rope_reencoder import RopeReencoder, inv_freq_table  # noqa: F401
