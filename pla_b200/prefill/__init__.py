"""Chunked-prefill operator surface (``pla.prefill``): ``flashqla`` (GDN) and ``flashkdapro`` (KDA)."""
