"""Control plane: slot ring, chunk and document metadata, RPC server, native index and lookup thread."""
