from .feetech import FeetechBus, decode_packet, encode_packet  # noqa: F401
