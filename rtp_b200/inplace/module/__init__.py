"""In-place rotated modules: the layer's single flat buffer itself travels around the ring through a small
staging chunk (no full-size receive buffer); compute and communication do not overlap."""
