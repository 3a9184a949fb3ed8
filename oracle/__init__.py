"""CPU oracle for the paged KV-cache path.  Test infrastructure only: the product package never imports it."""
