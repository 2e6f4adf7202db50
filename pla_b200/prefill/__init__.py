"""Chunked-prefill operator surface (``pla.prefill``): ``flashqla`` (GDN) and ``flashkdapro`` (KDA), plus the
causal conv that produces their packed inputs (``causal_conv``)."""
