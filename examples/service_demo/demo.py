"""Walk through the service API: health, upload two documents, list, get, infer, a streamed chat
completion (in-process engine only), delete, list.

    python -m daser_b200.service --engine native --tokenizer byte --store-path /tmp/d.store \
        --index-path /tmp/d.index --port 8080 &
    python examples/service_demo/demo.py --base-url http://127.0.0.1:8080

Counterpart of the reference's ``examples/service_demo/demo.py``.  With ``--engine native`` no
separate ``vllm serve`` is needed: the documents' chunks are stored by the in-process engine
and restored at their offsets when ``/infer`` builds a prompt from them.
"""

from __future__ import annotations

import argparse
import json

import httpx

DOC_A = ("The Blackwell generation keeps matrix accumulators in tensor memory next to the tensor "
         "cores, and moves operand tiles with an asynchronous copy engine. ") * 6
DOC_B = ("A retrieval-augmented prompt repeats the same document chunks across requests, so the keys "
         "and values of those chunks can be computed once and reused. ") * 6


def show(title: str, payload) -> None:
    print(f"--- {title}")
    print(json.dumps(payload, indent=2)[:1200])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--base-url", default="http://127.0.0.1:8080")
    args = ap.parse_args()
    with httpx.Client(base_url=args.base_url, timeout=300.0) as http:
        show("GET /health", http.get("/health").json())
        a = http.post("/documents", json={"title": "Blackwell notes", "text": DOC_A}).json()
        b = http.post("/documents", json={"title": "RAG notes", "text": DOC_B}).json()
        show("POST /documents (A)", a)
        show("POST /documents (B)", b)
        show("GET /documents", http.get("/documents").json())
        show(f"GET /documents/{a['doc_id']}", http.get(f"/documents/{a['doc_id']}").json())
        out = http.post("/infer", json={"doc_ids": [a["doc_id"], b["doc_id"]], "task": "Summarise both notes.",
                                        "gen_params": {"max_tokens": 16, "temperature": 0.0}}).json()
        show("POST /infer", out)
        if http.get("/v1/models").status_code == 200:  # the in-process engine also speaks vLLM's API
            print("--- POST /v1/chat/completions (stream): one event per token")
            body = {"messages": [{"role": "user", "content": "Which memory holds the accumulators?"}],
                    "max_tokens": 8, "temperature": 0.8, "seed": 7, "stream": True}
            with http.stream("POST", "/v1/chat/completions", json=body) as resp:
                for line in resp.iter_lines():
                    if line.startswith("data: {"):
                        choice = json.loads(line[6:])["choices"][0]
                        print(f"    {choice['delta']['content']!r} finish={choice['finish_reason']}")
        show(f"DELETE /documents/{a['doc_id']}", http.delete(f"/documents/{a['doc_id']}").json())
        show("GET /documents", http.get("/documents").json())
        print("--- GET /metrics (first lines)")
        print("\n".join(http.get("/metrics").text.splitlines()[:8]))


if __name__ == "__main__":
    main()
