"""REST front end: chunker, engine clients, the document / inference API, the OpenAI-style completions routes."""
