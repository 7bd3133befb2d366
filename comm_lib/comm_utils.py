"""Reference: comm_lib/comm_utils.py."""
from ultraattn_b200.parallel.comm import A2AComm, RingComm  # noqa: F401

RingCommOld = RingComm
RingCommNew = RingComm
