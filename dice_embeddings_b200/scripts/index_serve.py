"""Vector-database indexing and serving of trained entity embeddings.

``--index``: reads ``*_entity_embeddings.csv`` of a run and upserts the rows into a Qdrant collection (cosine
distance).  ``--serve``: FastAPI app with ``/api/search?q=<entity>&k=`` (nearest neighbours of a stored entity),
``/api/get?q=<entity>`` (its vector) and ``POST /api/search_batch``.  Qdrant is an optional dependency; when it is
not installed (or ``--backend local``) the same API is served from an in-process exact cosine index.
Reference: ``dicee/scripts/index_serve.py:19-150``.
"""
from __future__ import annotations

import argparse
import glob
import os
from typing import Dict, List, Optional

import numpy as np
import pandas as pd


class LocalCosineIndex:
    """Exact cosine search over a normalised matrix (stand-in for the vector database)."""

    def __init__(self, names: List[str], vectors: np.ndarray):
        self.names = list(names)
        self.pos: Dict[str, int] = {n: i for i, n in enumerate(self.names)}
        self.vectors = np.asarray(vectors, dtype=np.float32)
        n = np.linalg.norm(self.vectors, axis=1, keepdims=True)
        self.unit = self.vectors / np.maximum(n, 1e-12)

    def get(self, name: str) -> Optional[np.ndarray]:
        i = self.pos.get(name)
        return None if i is None else self.vectors[i]

    def search(self, name: str, k: int = 5):
        i = self.pos.get(name)
        if i is None:
            return []
        sims = self.unit @ self.unit[i]
        order = np.argsort(-sims)[: k + 1]
        return [{"hit": self.names[j], "score": float(sims[j])} for j in order if j != i][:k]


def load_entity_embeddings(path: str):
    files = sorted(glob.glob(os.path.join(path, "*_entity_embeddings.csv"))) or \
        sorted(glob.glob(os.path.join(path, "entity_embeddings.csv")))
    if not files:
        raise FileNotFoundError(f"no *_entity_embeddings.csv under {path}; train with --save_embeddings_as_csv")
    df = pd.read_csv(files[0], index_col=0)
    return [str(i) for i in df.index], df.values.astype(np.float32)


def index(path: str, collection: str, location: str = "localhost", port: int = 6333, batch: int = 1000):
    """Push the entity vectors of a run into a Qdrant collection."""
    from qdrant_client import QdrantClient
    from qdrant_client.http.models import Distance, PointStruct, VectorParams
    names, vecs = load_entity_embeddings(path)
    client = QdrantClient(host=location, port=port)
    if collection in [c.name for c in client.get_collections().collections]:
        client.delete_collection(collection)
    client.create_collection(collection, vectors_config=VectorParams(size=vecs.shape[1], distance=Distance.COSINE))
    for s in range(0, len(names), batch):
        pts = [PointStruct(id=s + i, vector=v.tolist(), payload={"name": n})
               for i, (n, v) in enumerate(zip(names[s:s + batch], vecs[s:s + batch]))]
        client.upsert(collection_name=collection, wait=True, points=pts)
    return len(names)


def create_app(path: str, collection: Optional[str] = None, backend: str = "local", location: str = "localhost",
               port: int = 6333):
    from fastapi import Body, FastAPI
    app = FastAPI(title="dice-embeddings-b200 vector search")
    names, vecs = load_entity_embeddings(path)
    local = LocalCosineIndex(names, vecs)
    client = None
    if backend == "qdrant":
        from qdrant_client import QdrantClient
        client = QdrantClient(host=location, port=port)

    def _search(q: str, k: int):
        if client is None:
            return local.search(q, k)
        v = local.get(q)
        if v is None:
            return []
        hits = client.search(collection_name=collection, query_vector=v.tolist(), limit=k + 1)
        return [{"hit": h.payload["name"], "score": h.score} for h in hits if h.payload["name"] != q][:k]

    @app.get("/")
    def root():
        return {"message": "use /api/search?q=<entity>&k=5, /api/get?q=<entity> or POST /api/search_batch"}

    @app.get("/api/search")
    def search(q: str, k: int = 5):
        return {"query": q, "results": _search(q, k)}

    @app.get("/api/get")
    def get(q: str):
        v = local.get(q)
        return {"query": q, "vector": None if v is None else v.tolist()}

    @app.post("/api/search_batch")
    def search_batch(b: dict = Body(...)):
        k = int(b.get("k", 5))
        return {"results": {q: _search(q, k) for q in b.get("queries", [])}}

    return app


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--path", type=str, required=True, help="run directory with *_entity_embeddings.csv")
    p.add_argument("--index", action="store_true")
    p.add_argument("--serve", action="store_true")
    p.add_argument("--collection", type=str, default="dice_embeddings")
    p.add_argument("--backend", choices=["local", "qdrant"], default="local")
    p.add_argument("--vdb_location", type=str, default="localhost")
    p.add_argument("--vdb_port", type=int, default=6333)
    p.add_argument("--host", type=str, default="0.0.0.0")
    p.add_argument("--port", type=int, default=8000)
    a = p.parse_args(argv)
    if a.index:
        n = index(a.path, a.collection, a.vdb_location, a.vdb_port)
        print(f"indexed {n} entities into {a.collection}")
    if a.serve:
        import uvicorn
        uvicorn.run(create_app(a.path, a.collection, a.backend, a.vdb_location, a.vdb_port), host=a.host, port=a.port)


if __name__ == "__main__":
    main()
