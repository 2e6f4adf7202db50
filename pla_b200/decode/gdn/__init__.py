"""GDN-only decode layouts (``pla.decode.gdn``)."""
