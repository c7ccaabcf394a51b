"""Wire format of the control-plane RPC: 4-byte big-endian length + msgpack map."""
