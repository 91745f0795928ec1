"""Asset packs: an ``assets.kv`` file declares the mesh / texture archives an environment needs and where they come
from; ``pull_pack`` fetches, verifies, extracts and links one (reference: noeira/assets/pack.mojo,
noeira/assets/resolve.mojo)."""
from .pack import PROVIDER_HF, PROVIDER_HTTPS, PROVIDER_NOEIRA, SCHEMA_VERSION, Pack, PackFile, load_packs, parse_packs
from .resolve import (Resolved, archive_path, cache_root, extract_dir, materialise, pack_bytes_on_disk, pack_status,
                      pull_pack, resolve_url)

__all__ = ["PROVIDER_HF", "PROVIDER_HTTPS", "PROVIDER_NOEIRA", "SCHEMA_VERSION", "Pack", "PackFile", "load_packs",
           "parse_packs", "Resolved", "archive_path", "cache_root", "extract_dir", "materialise", "pack_bytes_on_disk",
           "pack_status", "pull_pack", "resolve_url"]
