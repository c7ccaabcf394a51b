"""Operator's command line for a running control plane (over its Unix socket).

    python -m daser_b200.server.ctl [--socket-path /tmp/daser.sock] stats
    python -m daser_b200.server.ctl docs
    python -m daser_b200.server.ctl doc <doc_id>
    python -m daser_b200.server.ctl lookup <chunk_key> [<chunk_key> ...] [--model-id default]
    python -m daser_b200.server.ctl evict-chunk <chunk_key>
    python -m daser_b200.server.ctl evict-doc <doc_id>
    python -m daser_b200.server.ctl hello

Prints the reply as JSON; exits 1 on a transport or server error.  The reference has no such tool:
its state can only be inspected through the REST service's document routes.
"""

from __future__ import annotations

import argparse
import json
import sys
from typing import Optional, Sequence

from daser_b200.connector.ipc_client import IPCClientSync
from daser_b200.proto import frames


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="python -m daser_b200.server.ctl", description=__doc__.split("\n\n")[0])
    ap.add_argument("--socket-path", default="/tmp/daser.sock")
    ap.add_argument("--timeout", type=float, default=10.0)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("stats")
    sub.add_parser("hello")
    sub.add_parser("docs")
    p = sub.add_parser("doc")
    p.add_argument("doc_id")
    p = sub.add_parser("lookup")
    p.add_argument("keys", nargs="+")
    p.add_argument("--model-id", default="default")
    p = sub.add_parser("evict-chunk")
    p.add_argument("chunk_key")
    p = sub.add_parser("evict-doc")
    p.add_argument("doc_id")
    args = ap.parse_args(argv)
    payload = {
        "stats": lambda: {"op": frames.OP_STATS},
        "hello": lambda: {"op": frames.OP_HELLO, "geometry": {}},
        "docs": lambda: {"op": frames.OP_LIST_DOCS},
        "doc": lambda: {"op": frames.OP_GET_DOC, "doc_id": args.doc_id},
        "lookup": lambda: {"op": frames.OP_LOOKUP_CHUNKS, "keys": list(args.keys), "model_id": args.model_id},
        "evict-chunk": lambda: {"op": frames.OP_EVICT_CHUNK, "chunk_key": args.chunk_key},
        "evict-doc": lambda: {"op": frames.OP_EVICT_DOC, "doc_id": args.doc_id},
    }[args.cmd]()
    client = IPCClientSync(args.socket_path, timeout=args.timeout)
    try:
        reply = client.call(payload)
    except RuntimeError as exc:
        print(json.dumps({"error": str(exc)}), file=sys.stderr)
        return 1
    finally:
        client.close()
    json.dump(reply, sys.stdout, indent=1, sort_keys=True, default=str)
    sys.stdout.write("\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
