"""CPU oracle for the GQA attention path. Test infrastructure only: nothing in the product package may import this."""
